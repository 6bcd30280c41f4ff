// CPU walk of the persistent matvec kernel's work split (leviathan_b200/csrc/lev_chain_split.h):
// every tile is finished exactly once, every awaited count equals the arrivals that happen, and a
// finisher's rule for which record of a contributor to read names the record that was written.
#include <cstdio>
#include <cstdlib>
#include <map>
#include <set>
#include <tuple>
#include <vector>

#include "lev_chain_split.h"

static int fails = 0;
#define CHECK(c, ...)                     \
    do {                                  \
        if (!(c)) {                       \
            if (fails++ < 20) {           \
                printf("FAIL %s: ", #c);  \
                printf(__VA_ARGS__);      \
                printf("\n");             \
            }                             \
        }                                 \
    } while (0)

template <class T>
static void walk(int64_t tiles_, int spt_, int G_, int W_) {
    const T tiles = (T)tiles_, spt = (T)spt_, G = (T)G_, W = (T)W_;
    const T N = tiles * spt;
    std::vector<int> finished(tiles_, 0);
    std::map<std::pair<int64_t, int64_t>, int> block_arrivals, block_expected;  // (first block, tile)
    std::set<std::tuple<int64_t, int, int64_t>> block_records;                  // (block, which, tile) written
    for (T c = 0; c < G; c++) {
        const T cs = lev_split_lo<T>(N, c, G), ce = lev_split_lo<T>(N, c + 1, G), n = ce - cs;
        if (n == 0) continue;
        std::map<std::pair<int64_t, int64_t>, int> warp_arrivals, warp_expected;  // (ticket, tile)
        std::map<std::pair<int64_t, int>, int64_t> warp_records;                  // (warp, r) -> tile
        std::vector<T> block_done;  // tiles this block finishes at block level
        for (T w = 0; w < W; w++) {
            const T s = cs + lev_split_lo<T>(n, w, W), e = cs + lev_split_lo<T>(n, w + 1, W);
            if (s == e) continue;
            const T first_tile = s / spt;
            for (T q = s; q < e;) {
                const T tile = q / spt;
                T seg_end = (tile + 1) * spt;
                if (seg_end > e) seg_end = e;
                const bool whole = q == tile * spt && seg_end == (tile + 1) * spt;
                if (whole) {
                    finished[tile]++;
                } else {
                    const int r = tile == first_tile ? 0 : 1;
                    CHECK(warp_records.emplace(std::make_pair((int64_t)w, r), (int64_t)tile).second, "record reused: warp %d r %d", (int)w, r);
                    const T a = tile * spt > cs ? tile * spt : cs, b = (tile + 1) * spt < ce ? (tile + 1) * spt : ce;
                    // two tickets per warp: one for the tile that began in an earlier block, one for a tile that begins here
                    const int64_t ticket = 2 * (int64_t)lev_split_owner<T>(n, a - cs, W) + (tile * spt >= cs ? 1 : 0);
                    warp_arrivals[{ticket, (int64_t)tile}]++;
                    warp_expected[{ticket, (int64_t)tile}] = (int)lev_split_sharers<T>(n, a - cs, b - cs, W);
                }
                q = seg_end;
            }
        }
        std::set<int64_t> used_ticket;
        for (auto& kv : warp_arrivals) {
            CHECK(kv.second == warp_expected[kv.first], "warp arrivals %d expected %d (tiles %lld spt %d G %d W %d cta %d)", kv.second,
                  warp_expected[kv.first], (long long)tiles_, spt_, G_, W_, (int)c);
            CHECK(used_ticket.insert(kv.first.first).second, "ticket %lld used by two tiles", (long long)kv.first.first);
            // the finisher reads, for every contributor l, record (tile == s_l / spt ? 0 : 1)
            const T tile = (T)kv.first.second;
            const T a = tile * spt > cs ? tile * spt : cs, b = (tile + 1) * spt < ce ? (tile + 1) * spt : ce;
            const T l_first = lev_split_owner<T>(n, a - cs, W), l_last = lev_split_owner<T>(n, b - 1 - cs, W);
            for (T l = l_first; l <= l_last; l++) {
                const T s2 = cs + lev_split_lo<T>(n, l, W), e2 = cs + lev_split_lo<T>(n, l + 1, W);
                if (s2 == e2) continue;
                const int r = tile == s2 / spt ? 0 : 1;
                auto it = warp_records.find({(int64_t)l, r});
                CHECK(it != warp_records.end() && it->second == (int64_t)tile, "finisher would read a wrong record (warp %d)", (int)l);
            }
            block_done.push_back(tile);
        }
        for (T tile : block_done) {
            const T ta = tile * spt, tb = ta + spt;
            if (ta >= cs && tb <= ce) {
                finished[tile]++;
            } else {
                const T c0 = lev_split_owner<T>(N, ta, G);
                const int which = c == c0 ? 1 : 0;
                CHECK(block_records.insert({(int64_t)c, which, (int64_t)tile}).second, "block record reused");
                for (auto& t : block_records)
                    if (std::get<0>(t) == (int64_t)c && std::get<1>(t) == which) CHECK(std::get<2>(t) == (int64_t)tile, "two tiles in one block record");
                block_arrivals[{(int64_t)c0, (int64_t)tile}]++;
                block_expected[{(int64_t)c0, (int64_t)tile}] = (int)lev_split_sharers<T>(N, ta, tb, G);
            }
        }
    }
    std::set<int64_t> used_c0;
    for (auto& kv : block_arrivals) {
        CHECK(kv.second == block_expected[kv.first], "block arrivals %d expected %d (tiles %lld spt %d G %d W %d)", kv.second,
              block_expected[kv.first], (long long)tiles_, spt_, G_, W_);
        CHECK(used_c0.insert(kv.first.first).second, "ticket of block %lld used by two tiles", (long long)kv.first.first);
        const T tile = (T)kv.first.second, ta = tile * spt, tb = ta + spt;
        const T c0 = lev_split_owner<T>(N, ta, G), c1 = lev_split_owner<T>(N, tb - 1, G);
        for (T cc = c0; cc <= c1; cc++) {
            if (lev_split_lo<T>(N, cc, G) == lev_split_lo<T>(N, cc + 1, G)) continue;
            CHECK(block_records.count({(int64_t)cc, cc == c0 ? 1 : 0, (int64_t)tile}) == 1, "block finisher would read an unwritten record (block %d)", (int)cc);
        }
        finished[tile]++;
    }
    for (int64_t t = 0; t < tiles_; t++)
        CHECK(finished[t] == 1, "tile %lld finished %d times (tiles %lld spt %d G %d W %d)", (long long)t, finished[t], (long long)tiles_, spt_, G_, W_);
}

int main() {
    // owner() inverts lo()
    for (int64_t n = 1; n <= 300; n++)
        for (int parts : {1, 3, 8, 12, 16, 148})
            for (int64_t q = 0; q < n; q++) {
                const int64_t p = lev_split_owner<int64_t>(n, q, parts);
                CHECK(lev_split_lo<int64_t>(n, p, parts) <= q && q < lev_split_lo<int64_t>(n, p + 1, parts), "owner(%lld,%lld,%d)=%d", (long long)n, (long long)q, parts, (int)p);
                CHECK((int64_t)lev_split_owner<uint32_t>((uint32_t)n, (uint32_t)q, (uint32_t)parts) == p, "32-bit owner differs");
            }
    const int spts[] = {1, 3, 4, 11, 16, 22, 44, 48, 64};
    const int64_t tile_counts[] = {1, 2, 3, 7, 16, 35, 148, 149, 176, 256, 768, 1000, 16384};
    for (int spt : spts)
        for (int64_t tiles : tile_counts)
            for (int G : {1, 2, 7, 132, 148})
                for (int W : {4, 8, 12, 16}) {
                    if (tiles * spt > 400000) continue;
                    walk<int64_t>(tiles, spt, G, W);
                    walk<uint32_t>(tiles, spt, G, W);
                }
    // the largest op the kernel accepts: the 32-bit forms agree with the 64-bit ones at the edge
    for (uint32_t parts : {16u, 148u, 160u}) {
        const uint32_t n = lev_split_max_items(parts);
        for (uint32_t p = 0; p <= parts; p++)
            CHECK((int64_t)lev_split_lo<uint32_t>(n, p, parts) == lev_split_lo<int64_t>(n, p, parts), "32-bit lo overflows");
        for (uint32_t q : {0u, 1u, n / 3, n / 2, n - 2, n - 1})
            CHECK((int64_t)lev_split_owner<uint32_t>(n, q, parts) == lev_split_owner<int64_t>(n, q, parts), "32-bit owner overflows");
    }
    if (fails) {
        printf("%d failures\n", fails);
        return 1;
    }
    printf("ok\n");
    return 0;
}
