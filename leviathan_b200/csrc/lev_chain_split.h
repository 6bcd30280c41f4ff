// Work split of the persistent matvec kernel (lev_chain.cu), as plain integer functions that
// compile for the host too: tests/cpp/chain_split_check.cpp walks them on the CPU and checks that
// every 16-row tile is finished exactly once and that every count a thread waits for is the count
// of arrivals that really happen.
//
// An op is a run of K-steps (tile-major: tile * spt + step).  The grid splits the run into equal
// contiguous shares, one per thread block, and a block splits its share the same way over its
// compute warps.  A tile whose steps all belong to one warp is finished by that warp; a tile shared
// by several warps of a block is finished by the last of them to arrive (it adds the warps' partial
// sums in warp order); a tile shared by several blocks is finished by the last block to arrive (it
// adds the blocks' partial sums in block order).  Orders are fixed, so repeat runs give the same
// bits whoever arrives last.
#pragma once
#include <stdint.h>

#ifdef __CUDACC__
#define LEV_HD __host__ __device__ __forceinline__
#else
#define LEV_HD inline
#endif

// The kernel runs these in 32-bit unsigned arithmetic (n * parts stays below 2^32: the host side
// refuses larger ops), the CPU walk in 64-bit and in 32-bit.

// part p of `parts` owns items [n*p/parts, n*(p+1)/parts)
template <class T>
LEV_HD T lev_split_lo(T n, T p, T parts) { return n * p / parts; }

// the part that owns item q, 0 <= q < n
template <class T>
LEV_HD T lev_split_owner(T n, T q, T parts) { return ((q + 1) * parts - 1) / n; }

// parts that own at least one item of [a, b), 0 <= a < b <= n: every part in the owners' range when
// each part has an item, else one part per item (no part then has more than one)
template <class T>
LEV_HD T lev_split_sharers(T n, T a, T b, T parts) {
    if (n >= parts) return lev_split_owner<T>(n, b - 1, parts) - lev_split_owner<T>(n, a, parts) + 1;
    return b - a;
}

// largest K-step count of one op for which the 32-bit forms cannot overflow on `parts` parts
LEV_HD uint32_t lev_split_max_items(uint32_t parts) { return 0xffffffffu / (parts + 1u) - 1u; }
