#pragma once
// Prefetch into L2 across a kernel boundary. A decode step is a chain of short, dependent kernels, each of which streams a matrix it reads exactly once;
// between two of them (drain, launch, prologue, the first copies' round trip to device memory) the memory system idles. A kernel that is told what the
// next kernel will read first asks for those bytes with bulk prefetches (cp.async.bulk.prefetch.L2: no destination, no completion to wait for), so that the
// next kernel's first stages come out of L2. The description below is what a streaming GEMV of this backend reads first: the head of every block's row
// range (the blocks of a launch all start at the beginning of their own ranges), for one or two matrices of the same geometry, and optionally two linear
// ranges whose length depends on the decoder's position (the key and value rows of a layer).
#include <cstdint>

namespace dooms {
namespace cuda {

struct L2Prefetch {
    const uint8_t * mat[2];      // matrices of the next streaming GEMV (second: the up matrix of a fused gate/up), nullptr: none
    uint32_t row_bytes;          // bytes per matrix row
    int32_t rows_q, rows_r;      // the next launch's row split: block j owns rows_q + (j < rows_r) units of row_unit rows from unit j rows_q + min(j, rows_r)
    int32_t row_unit, grid;
    int32_t head_rows;           // rows at the start of each block's range to bring in
    int64_t rows;                // rows of the matrix
    const uint8_t * lin[2];      // linear ranges, nullptr: none
    uint32_t lin_bytes_per_pos;  // their length is (*pos) * lin_bytes_per_pos + lin_fixed_bytes
    uint32_t lin_fixed_bytes;
    const int32_t * pos;         // device word (the decoder's position), nullptr: only the fixed part
};

}  // namespace cuda

namespace dev {

__device__ __forceinline__ void bulk_prefetch_l2(const uint8_t * p, uint32_t bytes) {
    asm volatile("cp.async.bulk.prefetch.L2.global [%0], %1;" ::"l"(p), "r"(bytes) : "memory");
}

// [p, p + bytes) widened to 16-byte boundaries, in pieces of at most 32 KB.
__device__ __forceinline__ void prefetch_range_l2(const uint8_t * p, int64_t bytes) {
    const uint64_t a = reinterpret_cast<uint64_t>(p);
    const uint64_t lo = a & ~uint64_t(15), hi = (a + uint64_t(bytes) + 15u) & ~uint64_t(15);
    for (uint64_t q = lo; q < hi; q += 32768u) bulk_prefetch_l2(reinterpret_cast<const uint8_t *>(q), uint32_t(hi - q < 32768u ? hi - q : 32768u));
}

// This block's share of the prefetch, issued by the calling thread (one thread per block calls this).
__device__ __forceinline__ void l2_prefetch_issue(const cuda::L2Prefetch & h, int block, int nblocks) {
    if (h.mat[0]) {
        for (int j = block; j < h.grid; j += nblocks) {
            const int64_t r0 = (int64_t(j) * h.rows_q + (j < h.rows_r ? j : h.rows_r)) * h.row_unit;
            int64_t n = int64_t(h.rows_q + (j < h.rows_r ? 1 : 0)) * h.row_unit;
            if (n > h.rows - r0) n = h.rows - r0;
            if (n > h.head_rows) n = h.head_rows;
            if (n <= 0) continue;
            prefetch_range_l2(h.mat[0] + r0 * int64_t(h.row_bytes), n * int64_t(h.row_bytes));
            if (h.mat[1]) prefetch_range_l2(h.mat[1] + r0 * int64_t(h.row_bytes), n * int64_t(h.row_bytes));
        }
    }
    if (h.lin[0]) {
        const int64_t total = (h.pos ? int64_t(*h.pos) : 0) * int64_t(h.lin_bytes_per_pos) + int64_t(h.lin_fixed_bytes);
        const int64_t slice = ((total + nblocks - 1) / nblocks + 127) & ~int64_t(127);
        const int64_t off = int64_t(block) * slice;
        const int64_t len = total - off < slice ? total - off : slice;
        if (len > 0) {
            prefetch_range_l2(h.lin[0] + off, len);
            if (h.lin[1]) prefetch_range_l2(h.lin[1] + off, len);
        }
    }
}

}  // namespace dev
}  // namespace dooms
