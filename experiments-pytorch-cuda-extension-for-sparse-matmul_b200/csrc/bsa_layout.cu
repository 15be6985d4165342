// Device-side builder of the block layout metadata.
//
// Produces exactly the four tensors that SparseLayout._create_layout
// (reference sparse/layout.py:14-38) computes with torch ops on the host:
// row-ordered and column-ordered (idx, packed_pos) descriptor lists and their
// group offset tables.  Everything is integer work done with ballots and
// scans (no atomics), so the result is deterministic and bit-exact.
#include "bsa_common.cuh"

namespace bsa {
namespace {

constexpr int kLayoutThreads = 1024;
constexpr int kLayoutWarps = kLayoutThreads / 32;

// In-place inclusive scan of arr[0..n) by one thread block.
__device__ void block_inclusive_scan(int32_t* arr, int n, int32_t* warp_sums) {
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    int32_t carry = 0;
    for (int base = 0; base < n; base += kLayoutThreads) {
        const int i = base + tid;
        int32_t v = i < n ? arr[i] : 0;
#pragma unroll
        for (int d = 1; d < 32; d <<= 1) {
            int32_t o = __shfl_up_sync(0xffffffffu, v, d);
            if (lane >= d) v += o;
        }
        if (lane == 31) warp_sums[warp] = v;
        __syncthreads();
        if (warp == 0) {
            int32_t s = warp_sums[lane];
#pragma unroll
            for (int d = 1; d < 32; d <<= 1) {
                int32_t o = __shfl_up_sync(0xffffffffu, s, d);
                if (lane >= d) s += o;
            }
            warp_sums[lane] = s;  // inclusive sums of the warps
        }
        __syncthreads();
        const int32_t before = warp > 0 ? warp_sums[warp - 1] : 0;
        const int32_t total = warp_sums[kLayoutWarps - 1];
        if (i < n) arr[i] = carry + before + v;
        carry += total;
        __syncthreads();
    }
}

template <typename P>
__global__ void __launch_bounds__(kLayoutThreads)
layout_build_kernel(const P* __restrict__ pattern, int rows, int cols,
                    BlockDesc* __restrict__ row_blocks, int32_t* __restrict__ row_table,
                    BlockDesc* __restrict__ col_blocks, int32_t* __restrict__ col_table,
                    int32_t* __restrict__ nnz_out) {
    __shared__ int32_t warp_sums[kLayoutWarps];
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const unsigned lt_mask = (1u << lane) - 1u;

    // 1. per-row and per-column counts, stored one slot to the right so that
    //    the inclusive scan below yields the exclusive offsets.
    for (int r = warp; r < rows; r += kLayoutWarps) {
        int count = 0;
        for (int c0 = 0; c0 < cols; c0 += 32) {
            const int c = c0 + lane;
            const bool on = c < cols && pattern[(size_t)r * cols + c] != P(0);
            count += __popc(__ballot_sync(0xffffffffu, on));
        }
        if (lane == 0) row_table[r + 1] = count;
    }
    for (int c = tid; c < cols; c += kLayoutThreads) {
        int count = 0;
        for (int r = 0; r < rows; ++r) count += pattern[(size_t)r * cols + c] != P(0);
        col_table[c + 1] = count;
    }
    if (tid == 0) { row_table[0] = 0; col_table[0] = 0; }
    __syncthreads();

    // 2. offsets of the first block of every group.
    block_inclusive_scan(row_table + 1, rows, warp_sums);
    block_inclusive_scan(col_table + 1, cols, warp_sums);
    __syncthreads();

    // 3. row layout: blocks in (row, col) order; there idx equals the position.
    for (int r = warp; r < rows; r += kLayoutWarps) {
        int pos = row_table[r];
        for (int c0 = 0; c0 < cols; c0 += 32) {
            const int c = c0 + lane;
            const bool on = c < cols && pattern[(size_t)r * cols + c] != P(0);
            const unsigned ballot = __ballot_sync(0xffffffffu, on);
            if (on) {
                const int p = pos + __popc(ballot & lt_mask);
                row_blocks[p] = BlockDesc{p, (int32_t)(((uint32_t)r << 16) | (uint32_t)c)};
            }
            pos += __popc(ballot);
        }
    }
    __syncthreads();  // row_blocks written by this block are visible below

    // 4. column layout: blocks in (col, row) order; idx is looked up in the
    //    finished row layout by binary search on the column.
    for (int c = warp; c < cols; c += kLayoutWarps) {
        int pos = col_table[c];
        for (int r0 = 0; r0 < rows; r0 += 32) {
            const int r = r0 + lane;
            const bool on = r < rows && pattern[(size_t)r * cols + c] != P(0);
            const unsigned ballot = __ballot_sync(0xffffffffu, on);
            if (on) {
                int lo = row_table[r], hi = row_table[r + 1] - 1;
                while (lo < hi) {
                    const int mid = (lo + hi) >> 1;
                    if (row_blocks[mid].col() < c) lo = mid + 1; else hi = mid;
                }
                const int p = pos + __popc(ballot & lt_mask);
                col_blocks[p] = BlockDesc{lo, (int32_t)(((uint32_t)r << 16) | (uint32_t)c)};
            }
            pos += __popc(ballot);
        }
    }
    if (tid == 0) *nnz_out = row_table[rows];
}

}  // namespace
}  // namespace bsa

extern "C" int bsa_layout_build(const void* pattern, int pattern_dtype, int rows, int cols,
                                int32_t* row_blocks, int32_t* row_table,
                                int32_t* col_blocks, int32_t* col_table,
                                int32_t* nnz_out, void* stream) {
    using namespace bsa;
    if (!pattern || !row_blocks || !row_table || !col_blocks || !col_table || !nnz_out)
        return BSA_ERR_NULL_POINTER;
    if (rows <= 0 || cols <= 0) return BSA_ERR_BAD_SHAPE;
    if (rows > 65535 || cols > 65535) return BSA_ERR_TOO_LARGE;
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    BlockDesc* rb = reinterpret_cast<BlockDesc*>(row_blocks);
    BlockDesc* cb = reinterpret_cast<BlockDesc*>(col_blocks);
    switch (pattern_dtype) {
        case BSA_PATTERN_U8:
            layout_build_kernel<uint8_t><<<1, kLayoutThreads, 0, s>>>(
                static_cast<const uint8_t*>(pattern), rows, cols, rb, row_table, cb, col_table, nnz_out);
            break;
        case BSA_PATTERN_I32:
            layout_build_kernel<int32_t><<<1, kLayoutThreads, 0, s>>>(
                static_cast<const int32_t*>(pattern), rows, cols, rb, row_table, cb, col_table, nnz_out);
            break;
        case BSA_PATTERN_I64:
            layout_build_kernel<int64_t><<<1, kLayoutThreads, 0, s>>>(
                static_cast<const int64_t*>(pattern), rows, cols, rb, row_table, cb, col_table, nnz_out);
            break;
        case BSA_PATTERN_F32:
            layout_build_kernel<float><<<1, kLayoutThreads, 0, s>>>(
                static_cast<const float*>(pattern), rows, cols, rb, row_table, cb, col_table, nnz_out);
            break;
        default:
            return BSA_ERR_BAD_DTYPE;
    }
    return launch_status();
}
