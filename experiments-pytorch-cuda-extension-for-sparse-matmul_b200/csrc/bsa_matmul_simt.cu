// CUDA-core engine for the block-sparse matmul: every (mode, trans_a, trans_b)
// variant, every dtype and block size, fp32 accumulation.
//
// This engine is the exact-fp32 path (it keeps the 1e-4 tolerance for fp32
// inputs without any split) and the fallback for shapes the tcgen05 engine
// does not take.  It implements the *intended* semantics of the reference
// kernels sparse_smm_{sdd,dsd,dds}_32x32x32_kernel
// (sparse/native/sparse_smm_gpu.cu:22-267): the reference picks the wrong
// block coordinate for dsd with trans_a (:134,155) and dds with trans_b
// (:219,240) and never launches sdd with trans_a only (:287); here the K index
// is the block row for a transposed sparse A / plain sparse B and the block
// column otherwise, which is what the autograd table of sparse/matmul.py:30-50
// requires.
//
// One CTA of 256 threads computes a 32x32 output tile as a sum of 32x32x32
// sub-products staged through padded shared memory; operand sub-tiles are
// described by a base pointer and two strides, so transposition is a choice
// of strides.  All offsets are 64-bit.
#include <algorithm>

#include "bsa_common.cuh"

namespace bsa {
namespace {

constexpr int kTile = 32;
constexpr int kThreads = 256;

struct SubTile {
    size_t base;     // element offset of (0, 0)
    int64_t s_mn;    // stride along the M (for A) / N (for B) index
    int64_t s_k;     // stride along the K index
    int lim_mn;      // valid extent along M / N (<= 32)
    int lim_k;       // valid extent along K (<= 32)
};

template <typename T>
__device__ __forceinline__ void stage(const T* __restrict__ src, const SubTile& t, float (*dst)[kTile + 1]) {
    // dst[k][mn]; the thread-fast index follows the contiguous stride.
    const int tx = threadIdx.x & 31, ty = threadIdx.x >> 5;
    const bool k_fast = t.s_k == 1;
#pragma unroll
    for (int u = 0; u < kTile / 8; ++u) {
        const int k = k_fast ? tx : ty + 8 * u;
        const int mn = k_fast ? ty + 8 * u : tx;
        float v = 0.f;
        if (k < t.lim_k && mn < t.lim_mn) v = Scalar<T>::to_float(src[t.base + mn * t.s_mn + k * t.s_k]);
        dst[k][mn] = v;
    }
}

template <typename T>
__device__ __forceinline__ void accumulate(const T* __restrict__ a, const SubTile& ta,
                                           const T* __restrict__ b, const SubTile& tb,
                                           float (*sa)[kTile + 1], float (*sb)[kTile + 1],
                                           float (&acc)[2][2]) {
    __syncthreads();
    stage<T>(a, ta, sa);
    stage<T>(b, tb, sb);
    __syncthreads();
    const int r = (threadIdx.x >> 4) * 2, c = (threadIdx.x & 15) * 2;
#pragma unroll
    for (int k = 0; k < kTile; ++k) {
        const float a0 = sa[k][r], a1 = sa[k][r + 1];
        const float b0 = sb[k][c], b1 = sb[k][c + 1];
        acc[0][0] += a0 * b0; acc[0][1] += a0 * b1;
        acc[1][0] += a1 * b0; acc[1][1] += a1 * b1;
    }
}

struct Params {
    const void* a; const void* b; void* c;
    const BlockDesc* blocks; const int32_t* table;
    int64_t nnz, size_m, size_n, size_k;
    int block, trans_a, trans_b;
};

// SDD: grid (nnz * S * S, batches), S = ceil(block / 32).
template <typename T>
__global__ void __launch_bounds__(kThreads) sdd_kernel(const Params p) {
    __shared__ float sa[kTile][kTile + 1], sb[kTile][kTile + 1];
    const int B = p.block, S = (B + kTile - 1) / kTile;
    const int64_t bi = blockIdx.x / (S * S);
    const int sub = blockIdx.x % (S * S), si = sub / S, sj = sub % S;
    const int64_t z = blockIdx.y;
    const BlockDesc d = p.blocks[bi];
    const int64_t m0 = (int64_t)d.row() * B + si * kTile, n0 = (int64_t)d.col() * B + sj * kTile;
    // A descriptor is trusted neither for its position (a block beyond the dense operands reads as zero: the
    // limits below go to <= 0, as the TMA boxes of the tensor-core engine clip) nor for its rank (no write
    // outside the sparse tensor).
    const int lim_i = (int)min((int64_t)min(kTile, B - si * kTile), p.size_m - m0);
    const int lim_j = (int)min((int64_t)min(kTile, B - sj * kTile), p.size_n - n0);
    if (d.idx < 0 || d.idx >= p.nnz) return;
    const T* a = static_cast<const T*>(p.a) + z * p.size_m * p.size_k;
    const T* b = static_cast<const T*>(p.b) + z * p.size_k * p.size_n;
    float acc[2][2] = {};
    for (int64_t k0 = 0; k0 < p.size_k; k0 += kTile) {
        const int lim_k = (int)min((int64_t)kTile, p.size_k - k0);
        SubTile ta, tb;
        if (!p.trans_a) ta = {(size_t)(m0 * p.size_k + k0), p.size_k, 1, lim_i, lim_k};
        else            ta = {(size_t)(k0 * p.size_m + m0), 1, p.size_m, lim_i, lim_k};
        if (!p.trans_b) tb = {(size_t)(k0 * p.size_n + n0), 1, p.size_n, lim_j, lim_k};
        else            tb = {(size_t)(n0 * p.size_k + k0), p.size_k, 1, lim_j, lim_k};
        accumulate<T>(a, ta, b, tb, sa, sb, acc);
    }
    T* c = static_cast<T*>(p.c) + ((size_t)z * p.nnz + d.idx) * B * B;
    const int r = (threadIdx.x >> 4) * 2, cc = (threadIdx.x & 15) * 2;
#pragma unroll
    for (int u = 0; u < 2; ++u)
#pragma unroll
        for (int v = 0; v < 2; ++v)
            if (r + u < lim_i && cc + v < lim_j)
                c[(size_t)(si * kTile + r + u) * B + sj * kTile + cc + v] = Scalar<T>::from_float(acc[u][v]);
}

// DSD and DDS: grid (batches, tiles along M, tiles along N); the CTA walks the
// blocks of the group its output tile belongs to.  Along the sparse operand's
// grouped axis a tile is min(32, block) wide, so that it never spans two groups.
template <typename T, bool kSparseA>
__global__ void __launch_bounds__(kThreads) walk_kernel(const Params p) {
    __shared__ float sa[kTile][kTile + 1], sb[kTile][kTile + 1];
    const int B = p.block, KS = (B + kTile - 1) / kTile;
    const int64_t z = blockIdx.x;
    const int step_m = kSparseA ? min(kTile, B) : kTile, step_n = kSparseA ? kTile : min(kTile, B);
    const int64_t m0 = (int64_t)blockIdx.y * step_m, n0 = (int64_t)blockIdx.z * step_n;
    const int lim_i = (int)min((int64_t)step_m, p.size_m - m0), lim_j = (int)min((int64_t)step_n, p.size_n - n0);
    const int64_t walk_pos = kSparseA ? m0 : n0;          // position along the sparse operand's grouped axis
    const int g = (int)(walk_pos / B), sub = (int)(walk_pos % B);   // group and offset inside the block
    const int lim_sub = min(kTile, B - sub);
    const T* a = static_cast<const T*>(p.a) + (kSparseA ? (size_t)z * p.nnz * B * B : (size_t)z * p.size_m * p.size_k);
    const T* b = static_cast<const T*>(p.b) + (kSparseA ? (size_t)z * p.size_k * p.size_n : (size_t)z * p.nnz * B * B);
    float acc[2][2] = {};
    const int first = p.table[g], last = p.table[g + 1];
    for (int it = first; it < last; ++it) {
        const BlockDesc d = p.blocks[it];
        if (d.idx < 0 || d.idx >= p.nnz) continue;        // not a block of this sparse tensor (uniform for the CTA)
        const size_t blk = (size_t)d.idx * B * B;
        // block index along K: the coordinate of the block that is NOT the group
        int kb;
        if (kSparseA) kb = p.trans_a ? d.row() : d.col();
        else          kb = p.trans_b ? d.col() : d.row();
        for (int kk = 0; kk < KS; ++kk) {
            const int64_t k0 = (int64_t)kb * B + kk * kTile;
            // a block beyond the dense operand's inner extent contributes nothing (limit <= 0: nothing is read)
            const int lim_k = (int)min((int64_t)min(kTile, B - kk * kTile), p.size_k - k0);
            SubTile ta, tb;
            if (kSparseA) {
                if (!p.trans_a) ta = {blk + (size_t)sub * B + kk * kTile, B, 1, min(lim_i, lim_sub), lim_k};
                else            ta = {blk + (size_t)(kk * kTile) * B + sub, 1, B, min(lim_i, lim_sub), lim_k};
                if (!p.trans_b) tb = {(size_t)(k0 * p.size_n + n0), 1, p.size_n, lim_j, lim_k};
                else            tb = {(size_t)(n0 * p.size_k + k0), p.size_k, 1, lim_j, lim_k};
            } else {
                if (!p.trans_a) ta = {(size_t)(m0 * p.size_k + k0), p.size_k, 1, lim_i, lim_k};
                else            ta = {(size_t)(k0 * p.size_m + m0), 1, p.size_m, lim_i, lim_k};
                if (!p.trans_b) tb = {blk + (size_t)(kk * kTile) * B + sub, 1, B, min(lim_j, lim_sub), lim_k};
                else            tb = {blk + (size_t)sub * B + kk * kTile, B, 1, min(lim_j, lim_sub), lim_k};
            }
            accumulate<T>(a, ta, b, tb, sa, sb, acc);
        }
    }
    T* c = static_cast<T*>(p.c) + (size_t)z * p.size_m * p.size_n;
    const int r = (threadIdx.x >> 4) * 2, cc = (threadIdx.x & 15) * 2;
#pragma unroll
    for (int u = 0; u < 2; ++u)
#pragma unroll
        for (int v = 0; v < 2; ++v)
            if (r + u < lim_i && cc + v < lim_j)
                c[(size_t)(m0 + r + u) * p.size_n + n0 + cc + v] = Scalar<T>::from_float(acc[u][v]);
}

template <typename T>
int launch(const MatmulArgs& g) {
    Params p{g.a, g.b, g.c, g.blocks, g.table, g.nnz, g.size_m, g.size_n, g.size_k, g.block, g.trans_a, g.trans_b};
    if (g.mode == BSA_MODE_SDD) {
        if (g.nnz == 0) return BSA_OK;
        const int S = (g.block + kTile - 1) / kTile;
        const int64_t gx = g.nnz * S * S;
        if (gx > (int64_t)INT32_MAX || g.batches > 65535) return BSA_ERR_TOO_LARGE;
        sdd_kernel<T><<<dim3((unsigned)gx, (unsigned)g.batches), kThreads, 0, g.stream>>>(p);
    } else {
        const int step_m = g.mode == BSA_MODE_DSD ? std::min(kTile, g.block) : kTile;
        const int step_n = g.mode == BSA_MODE_DSD ? kTile : std::min(kTile, g.block);
        const int64_t gy = (g.size_m + step_m - 1) / step_m, gz = (g.size_n + step_n - 1) / step_n;
        if (gy > 65535 || gz > 65535) return BSA_ERR_TOO_LARGE;
        const dim3 grid((unsigned)g.batches, (unsigned)gy, (unsigned)gz);
        if (g.mode == BSA_MODE_DSD) walk_kernel<T, true><<<grid, kThreads, 0, g.stream>>>(p);
        else                        walk_kernel<T, false><<<grid, kThreads, 0, g.stream>>>(p);
    }
    return launch_status();
}

}  // namespace

int matmul_simt(const MatmulArgs& g) {
    switch (g.dtype) {
        case BSA_DTYPE_F32: return launch<float>(g);
        case BSA_DTYPE_F16: return launch<__half>(g);
        case BSA_DTYPE_BF16: return launch<__nv_bfloat16>(g);
        default: return BSA_ERR_BAD_DTYPE;
    }
}

}  // namespace bsa
