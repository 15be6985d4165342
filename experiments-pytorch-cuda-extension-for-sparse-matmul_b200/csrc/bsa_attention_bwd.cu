// Fused block-sparse attention backward (sm_100a only): dQ, dK, dV of
//   O = softmax_rows(scale * Q K^T + masks, restricted to the layout) V
// from Q, K, V, O, dO and the row log-sum-exp the forward kernel keeps, without the score,
// probability or score-gradient blocks ever travelling through HBM.  The reference composes the
// backward from its matmul in sdd / dsd mode (sparse/matmul.py:30-50 over sparse_smm_gpu.cu:22-183)
// and its softmax backward (sparse_softmax.cu:165-205), each step writing a [batch, nnz, block,
// block] tensor; this entry point has no counterpart there and exists beside the unfused operators.
//
// With D_i = sum_d dO_id O_id and, for every block (r, c) of the layout,
//   P = exp(scale * Q_r K_c^T - lse_r),  dP = dO_r V_c^T,  dS = scale * P o (dP - D_r):
//   dQ_r = sum_c dS K_c        dK_c = sum_r dS^T Q_r        dV_c = sum_r P^T dO_r.
// Three launches: a small kernel writes (lse in log2 units, D) per query row; then one kernel
// template runs twice:
//   by rows    item = block row r of a batch entry, resident pair X = (Q_r, dO_r), per block the
//              pair Y = (K_c, V_c):  T1 = X1 Y1^T = S, T2 = X2 Y2^T = dP, one operand tile dS,
//              one accumulator dQ += dS Y1.
//   by columns item = block column c (column layout), X = (K_c, V_c), Y = (Q_r, dO_r):
//              T1 = S^T, T2 = dP^T (keys on the TMEM lanes, queries along the columns, so lse and
//              D are per-column vectors, brought into shared memory with the block), two operand tiles
//              P^T and dS^T, two accumulators dV += P^T Y2 and dK += dS^T Y1.
// All products run on the tensor cores (tcgen05, fp32 accumulators in TMEM, 16-bit operand tiles
// of 64 x 64 in 128-byte-swizzled shared memory, loaded by TMA); the same shared-memory tile of Y
// serves as the K-major B operand of T and as the MN-major B operand of the accumulations.
// One CTA per SM with all 512 TMEM columns: T1 | T2 double buffered (columns 0-255), accumulators
// from column 256 (two sets where they fit, so that the next item accumulates while an item is
// stored).  Warp roles (15 warps):
//   warps 0-7   two compute warpgroups taking alternate blocks: tcgen05.ld of T1 and T2 (16x256b
//               shape: a lane owns 2 rows x 16 columns), exp2, the dS formula, masks, 32-bit
//               stores into the swizzled operand tiles (a ring of 2 or 4 buffers); the groups
//               convert and store the accumulators of alternate items while the other one goes on.
//   warp 8      TMA producer: the item's X pair, every block's Y pair and, by columns, the 512
//               bytes of (lse, D) of the block's query rows (ring of 4 or 8 stages)
//   warps 9-12  issuers of T1 / T2 of the even / odd blocks (a thread issues one tcgen05.mma or
//               commit per ~100 cycles whatever its size)
//   warps 13-14 issuers of the accumulations: by columns one per output (dV, dK); by rows with
//               head dim 64 the K-steps 0-1 / 2-3 of dQ into two partial accumulators that the
//               epilogue adds; their commits per block free the Y stage and the operand tiles.
// Measured at seq 4096, 12 blocks per row, head dim 64: about 1000 cycles per block and SM by
// rows, 1300 by columns, whichever way the roles are cut (one or two issuers per product, 2 or 4
// operand buffers, 4 or 8 stages, one or two accumulator sets: within 5 %).  A 64 x 64 x 16 MMA
// reads 4 KB of operands from shared memory; the 12 (by rows) or 16 (by columns) of a block plus
// the TMA and operand-tile writes move 72 / 96 KB per block through a 128 B / cycle port, i.e.
// 560 / 750 cycles: the kernels sit at 55-60 % of that bound, like the forward kernel.
// Loops are warp-uniform with an elected lane around the TMA / tcgen05 instructions.  All waits are
// bounded (BSA_ERR_DEVICE_TIMEOUT in the workspace word).
#include <type_traits>

#include "bsa_tc_common.cuh"

namespace bsa {
namespace {

constexpr int kBwdTmemCols = 512;
constexpr int kBwdAccCol0 = 256;
constexpr int kBwdStatBytes = kTile * 8;      // (lse2, D) of the 64 query rows of a block
constexpr int kBwdMaxRing = 8;              // Y stages: a power of two, chosen per launch (BwdParams::ring)
constexpr float kLog2e = 1.4426950408889634f;

struct __align__(8) BwdBarriers {
    uint64_t x_full[2], x_empty[2];
    uint64_t y_full[kBwdMaxRing];
    uint64_t out_done[kBwdMaxRing];    // the accumulation MMAs of a block have retired: Y stage and operand tiles are free
    uint64_t t_full[2], t_empty[2];
    uint64_t op_full[4];            // the operand tile(s) of a block are written
    uint64_t o_full[2], o_empty[2];   // indexed by the parity of the item: each is waited on by one compute group only
    uint64_t drain;
    uint32_t tmem_base;
    int abort_flag;
};

struct BwdParams {
    const BlockDesc* blocks;   // row layout (by rows) or column layout (by columns)
    const int32_t* table;
    uint32_t* status;
    int nnz, groups, batches;
    int chunks, items;         // chunks = 1 (kept for the shared cursor)
    int stride_z, stride_rem;
    int seq_q, seq_k, head_dim, dtiles;
    int xbufs;                 // X pairs in shared memory (1 or 2)
    int opbufs, op_shift;      // operand tile buffers (2 or 4) and their log2: block s writes buffer s % opbufs once
                               // the accumulation MMAs of block s - opbufs have retired
    int parts;                 // partial accumulators per output (1 or 2), added up by the epilogue
    int out_issuers;           // warps issuing the accumulations (1 or 2)
    int obufs;                 // accumulator sets (1 or 2): with 2 the next item accumulates while an item is stored
    int ring, ring_shift;      // Y stages and their log2: a block holds its stage from the TMA request until its
                               // accumulation MMAs have retired, so the depth bounds the blocks in flight
    float scale, scale_log2;
    int causal;
    int quadrants;             // 1: descriptor idx = 4-bit mask of the block's 32 x 32 quadrants in the layout
                               // (bit 2 * row_half + col_half), the others are masked like causal / padded scores
    const uint8_t* kpm;
    int kpm_div;
    long long kpm_stride;
    const float2* stats;       // per query row: (lse * log2(e), or +inf for a row without scores; D)
    // head dim 64: the kernel by rows computes the statistics of its own rows from these and writes them to
    // `stats_out` for the kernel by columns (no statistics launch)
    const uint16_t* o;
    const uint16_t* dout;
    const float* lse;
    float2* stats_out;
    uint16_t* out0;            // by rows: dQ; by columns: dV
    uint16_t* out1;            // by columns: dK
    uint32_t idesc_t, idesc_acc;
};

// (lse in log2 units, D_i = sum_d dO_id O_id) per query row; one group of head_dim / 8 lanes per row.
template <bool BF16>
__global__ void __launch_bounds__(256)
attention_backward_stats_kernel(const uint16_t* __restrict__ o, const uint16_t* __restrict__ dout,
                                const float* __restrict__ lse, float2* __restrict__ stats,
                                long long rows, int head_dim) {
    const int lanes = head_dim / 8;                           // 8 or 16
    const long long row = ((long long)blockIdx.x * blockDim.x + threadIdx.x) / lanes;
    const int part = (int)(threadIdx.x % lanes);
    float acc = 0.f;
    if (row < rows) {
        const uint4 a = *reinterpret_cast<const uint4*>(o + row * head_dim + part * 8);
        const uint4 b = *reinterpret_cast<const uint4*>(dout + row * head_dim + part * 8);
        const uint32_t aw[4] = {a.x, a.y, a.z, a.w}, bw[4] = {b.x, b.y, b.z, b.w};
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            float2 fa, fb;
            if (BF16) {
                fa = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&aw[i]));
                fb = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&bw[i]));
            } else {
                fa = __half22float2(*reinterpret_cast<const __half2*>(&aw[i]));
                fb = __half22float2(*reinterpret_cast<const __half2*>(&bw[i]));
            }
            acc = fmaf(fa.x, fb.x, acc);
            acc = fmaf(fa.y, fb.y, acc);
        }
    }
    for (int d = lanes >> 1; d > 0; d >>= 1) acc += __shfl_xor_sync(0xffffffffu, acc, d);
    if (row < rows && part == 0) {
        const float l = lse[row];
        stats[row] = make_float2(l == -INFINITY ? INFINITY : l * kLog2e, acc);
    }
}

// Sum over 16 consecutive head-dim columns of dO * O (two 16-byte loads from each).
template <bool BF16>
__device__ __forceinline__ float dot16(const uint16_t* __restrict__ a, const uint16_t* __restrict__ b) {
    float acc = 0.f;
#pragma unroll
    for (int h = 0; h < 2; ++h) {
        const uint4 x = *reinterpret_cast<const uint4*>(a + 8 * h), y = *reinterpret_cast<const uint4*>(b + 8 * h);
        const uint32_t xw[4] = {x.x, x.y, x.z, x.w}, yw[4] = {y.x, y.y, y.z, y.w};
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            float2 fa, fb;
            if (BF16) {
                fa = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&xw[i]));
                fb = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&yw[i]));
            } else {
                fa = __half22float2(*reinterpret_cast<const __half2*>(&xw[i]));
                fb = __half22float2(*reinterpret_cast<const __half2*>(&yw[i]));
            }
            acc = fmaf(fa.x, fb.x, acc);
            acc = fmaf(fa.y, fb.y, acc);
        }
    }
    return acc;
}

// Warp roles.  The compute warpgroups come first (a warp reads the TMEM sub-partition warp % 4).
constexpr int kBwdProducerWarp = 8;
constexpr int kBwdFirstTWarp = 9;           // 9: T1 of even blocks, 10: T1 odd, 11: T2 even, 12: T2 odd
constexpr int kBwdFirstOutWarp = 13;        // 13: first accumulator, 14 (by columns): second accumulator
template <bool COL> constexpr int bwd_warps() { return 15; }

template <bool COL, bool BF16, bool MASKED>
__global__ void __launch_bounds__(bwd_warps<COL>() * 32, 1)
attention_backward_kernel(const __grid_constant__ CUtensorMap map_x1, const __grid_constant__ CUtensorMap map_x2,
                          const __grid_constant__ CUtensorMap map_y1, const __grid_constant__ CUtensorMap map_y2,
                          const BwdParams p) {
    extern __shared__ uint8_t smem_raw[];
    uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~(uintptr_t)1023);
    constexpr int kOpTiles = COL ? 2 : 1;                  // operand tiles per block
    constexpr int kOuts = COL ? 2 : 1;                     // outputs (accumulators per set, without partials)
    const int set_bytes = p.dtiles * kTileBytes;            // one 64-row tile set of Q / K / V / dO
    uint8_t* x_smem = smem;                                 // [xbufs][2][set]
    uint8_t* y_smem = x_smem + p.xbufs * 2 * set_bytes;     // [ring][2][set]
    uint8_t* op_smem = y_smem + p.ring * 2 * set_bytes;     // [opbufs][kOpTiles] tiles
    uint8_t* st_smem = op_smem + p.opbufs * kOpTiles * kTileBytes; // by columns: [ring] x 64 float2 (lse2, D) of the block's query rows
    BwdBarriers* bars = reinterpret_cast<BwdBarriers*>(st_smem + (COL ? p.ring * kBwdStatBytes : 0));
    int* abort_flag = &bars->abort_flag;

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int ring_mask = p.ring - 1;

    if (threadIdx.x == 0) {
        for (int s = 0; s < 2; ++s) {
            mbar_init(&bars->x_full[s], 1); mbar_init(&bars->x_empty[s], 4);
            mbar_init(&bars->t_full[s], 2); mbar_init(&bars->t_empty[s], 4);
        }
        for (int s = 0; s < 4; ++s) mbar_init(&bars->op_full[s], 4);
        for (int s = 0; s < kBwdMaxRing; ++s) { mbar_init(&bars->y_full[s], 1); mbar_init(&bars->out_done[s], (uint32_t)p.out_issuers); }
        for (int s = 0; s < 2; ++s) { mbar_init(&bars->o_full[s], (uint32_t)p.out_issuers); mbar_init(&bars->o_empty[s], 4); }
        mbar_init(&bars->drain, (uint32_t)(4 + p.out_issuers));
        bars->abort_flag = 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
        fence_async_shared();
    }
    if (warp == kBwdProducerWarp) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;"
                     ::"r"(smem_u32(&bars->tmem_base)), "r"((uint32_t)kBwdTmemCols) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem_base = *(volatile uint32_t*)&bars->tmem_base;

    if (warp == kBwdProducerWarp) {
        // ------------------------------------------------------------ TMA producer
        int y_no = 0, x_no = 0;
        bool ok = true;
        Cursor cur;
        cur.init(p, 0, true);
        BlockDesc pre = cur.valid() ? load_first_chunk(p.blocks, cur.first, cur.count, lane) : BlockDesc{0, 0};
        while (ok && cur.valid()) {
            BlockDesc pre_next{0, 0};
            if (cur.has_next()) pre_next = load_first_chunk(p.blocks, cur.next_first(), cur.next_count(), lane);
            const int n = cur.count;
            if (n > 0) {
                const int xb = x_no & (p.xbufs - 1);
                const uint32_t use = (uint32_t)(p.xbufs == 2 ? x_no >> 1 : x_no);
                ok = __all_sync(0xffffffffu, mbar_wait(&bars->x_empty[xb], (use & 1u) ^ 1u, abort_flag, p.status)) != 0;
                if (ok && elect_one()) {
                    mbar_expect_tx(&bars->x_full[xb], (uint32_t)(2 * set_bytes));
                    for (int t = 0; t < p.dtiles; ++t) {
                        tma_load_3d(x_smem + (xb * 2 + 0) * set_bytes + t * kTileBytes, &map_x1, &bars->x_full[xb], t * kTile, cur.g * kTile, cur.z);
                        tma_load_3d(x_smem + (xb * 2 + 1) * set_bytes + t * kTileBytes, &map_x2, &bars->x_full[xb], t * kTile, cur.g * kTile, cur.z);
                    }
                }
                __syncwarp();
                ++x_no;
                DescWindow win;
                win.begin(p.blocks, cur.first, cur.count, pre, lane);
                for (int j = 0; ok && j < n; ++j, ++y_no) {
                    const BlockDesc d = win.get(p.blocks, cur.first, cur.count, j, lane);
                    const int other = COL ? d.row() : d.col();
                    const int stage = y_no & ring_mask;
                    ok = __all_sync(0xffffffffu, mbar_wait(&bars->out_done[stage], ((uint32_t)(y_no >> p.ring_shift) & 1u) ^ 1u,
                                                           abort_flag, p.status)) != 0;
                    if (ok && elect_one()) {
                        uint64_t* full = &bars->y_full[stage];
                        mbar_expect_tx(full, (uint32_t)(2 * set_bytes + (COL ? kBwdStatBytes : 0)));
                        for (int t = 0; t < p.dtiles; ++t) {
                            tma_load_3d(y_smem + (stage * 2 + 0) * set_bytes + t * kTileBytes, &map_y1, full, t * kTile, other * kTile, cur.z);
                            tma_load_3d(y_smem + (stage * 2 + 1) * set_bytes + t * kTileBytes, &map_y2, full, t * kTile, other * kTile, cur.z);
                        }
                        if (COL)
                            bulk_load_1d(st_smem + stage * kBwdStatBytes,
                                         p.stats + (size_t)cur.z * p.seq_q + (size_t)other * kTile, kBwdStatBytes, full);
                    }
                    __syncwarp();
                }
            }
            pre = pre_next;
            cur.advance();
        }
        if (lane == 0 && *(volatile int*)abort_flag) {
            let_copies_land();      // (issued by this warp; see the helper)
        }
        __syncwarp();
    } else if (warp >= kBwdFirstTWarp && warp < kBwdFirstOutWarp) {
        // ------------------------------------------------------------ issuers of T1 = X1 Y1^T and T2 = X2 Y2^T
        // Four warps: product `which` of the blocks with number s & 1 == par (T buffer par).  A thread
        // issues one tcgen05.mma per ~100 cycles, so the 8 (head dim 64) MMAs + 2 commits of a block
        // would otherwise cost one issuer 1000 cycles per block.
        const int which = (warp - kBwdFirstTWarp) >> 1, par = (warp - kBwdFirstTWarp) & 1;
        int s_no = 0, x_no = 0;
        bool ok = true;
        Cursor cur;
        cur.init(p, 0, true);
        for (; ok && cur.valid(); cur.advance()) {
            const int n = cur.count;
            if (n == 0) continue;
            const int xb = x_no & (p.xbufs - 1);
            ok = __all_sync(0xffffffffu, mbar_wait(&bars->x_full[xb], (uint32_t)(p.xbufs == 2 ? x_no >> 1 : x_no) & 1u,
                                                   abort_flag, p.status)) != 0;
            if (!ok) break;
            const int s_end = s_no + n;
            for (int s = s_no + ((par - s_no) & 1); s < s_end; s += 2) {
                const int stage = s & ring_mask;
                ok = __all_sync(0xffffffffu, mbar_wait(&bars->y_full[stage], (uint32_t)(s >> p.ring_shift) & 1u, abort_flag, p.status)) != 0;
                if (ok) ok = __all_sync(0xffffffffu, mbar_wait(&bars->t_empty[par], ((uint32_t)(s >> 1) & 1u) ^ 1u, abort_flag, p.status)) != 0;
                if (!ok) break;
                tc_fence_after();
                const uint32_t d = tmem_base + (uint32_t)(par * 2 * kTile + which * kTile);
                if (elect_one()) {
                    for (int t = 0; t < p.dtiles; ++t) {
                        const uint64_t da = make_tile_desc(smem_u32(x_smem + (xb * 2 + which) * set_bytes + t * kTileBytes), false);
                        const uint64_t db = make_tile_desc(smem_u32(y_smem + (stage * 2 + which) * set_bytes + t * kTileBytes), false);
#pragma unroll
                        for (int kk = 0; kk < kTile / 16; ++kk)
                            tc_mma_f16(d, da + (uint64_t)(kk * 2), db + (uint64_t)(kk * 2), p.idesc_t, (t > 0 || kk > 0) ? 1u : 0u);
                    }
                    tc_commit(&bars->t_full[par]);
                }
                __syncwarp();
            }
            if (!ok) break;
            if (elect_one()) tc_commit(&bars->x_empty[xb]);       // this issuer's reads of the X pair have been issued
            __syncwarp();
            s_no = s_end;
            ++x_no;
        }
        // All MMAs issued by the elected lane (the same one every time) must have retired before TMEM is freed.
        if (elect_one()) {
            tc_commit(&bars->drain);
            mbar_wait(&bars->drain, 0, abort_flag, p.status);
        }
        __syncwarp();
    } else if (warp >= kBwdFirstOutWarp) {
        // ------------------------------------------------------------ issuers of the accumulations
        // By columns: warp 13 dV += P^T Y2, warp 14 dK += dS^T Y1.  By rows: dQ += dS Y1; with two partial
        // accumulators warp 13 issues K-steps 0, 1 into the first and warp 14 K-steps 2, 3 into the second
        // (4 MMAs and up to 2 commits per block cost one thread 400-500 cycles).  Accumulator set o_no % obufs.
        const int w = warp - kBwdFirstOutWarp;
        if (w < p.out_issuers) {
            const int kk0 = (!COL && p.out_issuers == 2) ? 2 * w : 0;          // this issuer's K-steps
            const int kk1 = (!COL && p.out_issuers == 2) ? 2 * w + 2 : kTile / 16;
            int s_no = 0, o_no = 0;
            bool ok = true;
            Cursor cur;
            cur.init(p, 0, true);
            for (; ok && cur.valid(); cur.advance()) {
                const int n = cur.count;
                if (n == 0) continue;
                const int ob_acc = o_no & (p.obufs - 1);          // accumulator set of this item
                // accumulator of this issuer: set, then output (by columns) or partial (by rows)
                const uint32_t d = tmem_base + (uint32_t)(kBwdAccCol0 + ((ob_acc * kOuts + (COL ? w : 0)) * p.parts + (COL ? 0 : (kk0 >> 1) & (p.parts - 1))) * p.head_dim);
                for (int j = 0; ok && j < n; ++j) {
                    const int s = s_no + j, stage = s & ring_mask, ob = s & (p.opbufs - 1);
                    // the accumulator set is free once the item that used it last (obufs items ago) has been
                    // read out; that item's barrier is the one of its parity
                    if (j == 0 && o_no >= p.obufs) {
                        const int prev = o_no - p.obufs;
                        ok = __all_sync(0xffffffffu, mbar_wait(&bars->o_empty[prev & 1], (uint32_t)(prev >> 1) & 1u, abort_flag, p.status)) != 0;
                    }
                    if (ok) ok = __all_sync(0xffffffffu, mbar_wait(&bars->y_full[stage], (uint32_t)(s >> p.ring_shift) & 1u, abort_flag, p.status)) != 0;
                    if (ok) ok = __all_sync(0xffffffffu, mbar_wait(&bars->op_full[ob], (uint32_t)(s >> p.op_shift) & 1u, abort_flag, p.status)) != 0;
                    if (!ok) break;
                    tc_fence_after();
                    if (elect_one()) {
                        // A = operand tile (K-major), B = a Y tile set with N = head_dim contiguous
                        const uint64_t a = make_tile_desc(smem_u32(op_smem + (ob * kOpTiles + (COL ? w : 0)) * kTileBytes), false);
                        const int ysel = COL ? 1 - w : 0;             // dV reads Y2 (dO), dK and dQ read Y1
                        const uint64_t b = make_tile_desc(smem_u32(y_smem + (stage * 2 + ysel) * set_bytes), true);
                        for (int kk = kk0; kk < kk1; ++kk)
                            tc_mma_f16(d, a + (uint64_t)(kk * 2), b + (uint64_t)(kk * (2048 >> 4)), p.idesc_acc,
                                       (j > 0 || kk > kk0) ? 1u : 0u);
                        tc_commit(&bars->out_done[stage]);
                        if (j == n - 1) tc_commit(&bars->o_full[o_no & 1]);
                    }
                    __syncwarp();
                }
                s_no += n;
                ++o_no;
            }
            if (elect_one()) {
                tc_commit(&bars->drain);
                mbar_wait(&bars->drain, 0, abort_flag, p.status);
            }
        }
        __syncwarp();
    } else {
        // ------------------------------------------------------------ compute warpgroups
        // Group g takes the blocks with number s & 1 == g (T buffer g, operand buffer g).
        const int wg = warp >> 2;
        const int quad = warp & 3;                  // TMEM sub-partition this warp may read
        const int q4 = lane & 3;                    // position in the quad: columns 8u + 2 * q4 + {0, 1}
        const int row_a = quad * 16 + (lane >> 2);  // this lane's two rows of the 64-row tile: row_a, row_a + 8
        const uint32_t lane_field = (uint32_t)(quad * 32) << 16;
        const bool masked_op = MASKED && (p.causal != 0 || p.kpm != nullptr || p.quadrants != 0);
        const float c2 = p.scale_log2, sc = p.scale;
        const int out_rows = COL ? p.seq_k : p.seq_q;
        int s_no = 0, o_no = 0;
        bool ok = true;
        Cursor cur;
        cur.init(p, 0, true);
        BlockDesc pre = cur.valid() ? load_first_chunk(p.blocks, cur.first, cur.count, lane) : BlockDesc{0, 0};
        while (ok && cur.valid()) {
            BlockDesc pre_next{0, 0};
            if (cur.has_next()) pre_next = load_first_chunk(p.blocks, cur.next_first(), cur.next_count(), lane);
            const int n = cur.count;
            const size_t out_a = ((size_t)cur.z * out_rows + (size_t)cur.g * kTile + row_a) * p.head_dim;
            const size_t out_b = out_a + (size_t)8 * p.head_dim;
            if (n == 0) {
                // a group without blocks: zero gradient rows
                if (wg == 0) {
                    for (int c = q4 * 8; c < p.head_dim; c += 32) {
                        *reinterpret_cast<uint4*>(p.out0 + out_a + c) = make_uint4(0u, 0u, 0u, 0u);
                        *reinterpret_cast<uint4*>(p.out0 + out_b + c) = make_uint4(0u, 0u, 0u, 0u);
                        if (COL) {
                            *reinterpret_cast<uint4*>(p.out1 + out_a + c) = make_uint4(0u, 0u, 0u, 0u);
                            *reinterpret_cast<uint4*>(p.out1 + out_b + c) = make_uint4(0u, 0u, 0u, 0u);
                        }
                    }
                }
            } else {
                const uint8_t* kpm_row = (MASKED && p.kpm) ? p.kpm + (size_t)(cur.z / p.kpm_div) * p.kpm_stride : nullptr;
                const int pos_a = cur.g * kTile + row_a;         // by rows: query position; by columns: key position
                const float2* stats_z = p.stats + (size_t)cur.z * p.seq_q;
                // by rows: the statistics of this lane's two query rows
                float2 st_a = make_float2(0.f, 0.f), st_b = st_a;
                if (!COL) { st_a = stats_z[pos_a]; st_b = stats_z[pos_a + 8]; }
                // by columns: a whole key row is padding or not
                bool pad_a = false, pad_b = false;
                if (COL && MASKED && kpm_row) { pad_a = kpm_row[pos_a] != 0; pad_b = kpm_row[pos_a + 8] != 0; }
                DescWindow win;
                win.begin(p.blocks, cur.first, cur.count, pre, lane);
                const uint32_t op_row = (uint32_t)(row_a * 128 + 4 * q4), op_xor = (uint32_t)(row_a & 7);
                const int t_first = (wg - s_no) & 1;            // this group's first block of the item
                for (int t = t_first; ok && t < n; t += 2) {
                    const int s = s_no + t, tb = s & 1;
                    // (the block's descriptor is needed for the masks only; fetching it from the window costs the
                    // compute warps two shuffles and the window's registers per block)
                    BlockDesc d{0, 0};
                    if (MASKED) d = win.get(p.blocks, cur.first, cur.count, t, lane);
                    const int other = COL ? d.row() : d.col();
                    // quadrant masks: is the half u < 4 / u >= 4 of this lane's 16 columns inside the layout?
                    // By rows the lane's rows are queries (row half quad / 2) and u / 4 the key half; by
                    // columns the lane's rows are keys (column half quad / 2) and u / 4 the query (row) half.
                    bool sub_lo = true, sub_hi = true;
                    if (MASKED && p.quadrants) {
                        const uint32_t bits = (uint32_t)d.idx;
                        const int h = quad >> 1;
                        sub_lo = COL ? ((bits >> h) & 1u) != 0 : ((bits >> (2 * h)) & 1u) != 0;
                        sub_hi = COL ? ((bits >> (2 + h)) & 1u) != 0 : ((bits >> (2 * h + 1)) & 1u) != 0;
                    }
                    ok = __all_sync(0xffffffffu, mbar_wait(&bars->t_full[tb], (uint32_t)(s >> 1) & 1u, abort_flag, p.status)) != 0;
                    if (!ok) break;
                    tc_fence_after();
                    uint32_t r1[32], r2[32];
                    tc_ld_16x256b_x8(tmem_base + lane_field + (uint32_t)(tb * 2 * kTile), r1);
                    tc_ld_16x256b_x8(tmem_base + lane_field + (uint32_t)(tb * 2 * kTile + kTile), r2);
                    // by columns: (lse2, D) of this lane's 16 query columns, brought into the block's stage by
                    // the producer: cs[u] = those of column 8u + 2 q4 and of column 8u + 2 q4 + 1
                    float4 cs[8];
                    if (COL) {
                        const int stage = s & ring_mask;
                        ok = __all_sync(0xffffffffu, mbar_wait(&bars->y_full[stage], (uint32_t)(s >> p.ring_shift) & 1u, abort_flag, p.status)) != 0;
                        if (!ok) break;
                        const float4* src = reinterpret_cast<const float4*>(st_smem + stage * kBwdStatBytes) + q4;
#pragma unroll
                        for (int u = 0; u < 8; ++u) cs[u] = src[4 * u];        // 8 columns = 4 float4 apart
                    }
                    tc_wait_ld();
                    release_accumulator(&bars->t_empty[tb], lane);
                    // the operand tiles of this buffer must have been read by the MMAs of block s - opbufs
                    const int ob = s & (p.opbufs - 1);
                    if (s >= p.opbufs) {
                        const int sp = s - p.opbufs;
                        ok = __all_sync(0xffffffffu, mbar_wait(&bars->out_done[sp & ring_mask],
                                                               (uint32_t)(sp >> p.ring_shift) & 1u, abort_flag, p.status)) != 0;
                        if (!ok) break;
                    }
                    const uint32_t tile0 = smem_u32(op_smem + (ob * kOpTiles) * kTileBytes) + op_row;
                    const int other0 = other * kTile + 2 * q4;          // position of column u = 0, e = 0
                    // Does any lane of the warp have a masked element in this block?  Most blocks of a causal
                    // or padded problem have none and take the plain code (the element-wise tests cost the
                    // compute warps half as many instructions again).
                    bool need = false;
                    uint32_t padbits = 0u;          // by rows: bit 2u + e = key column 8u + 2 q4 + e is padding
                    if (MASKED && masked_op) {
                        bool lane_need = !(sub_lo && sub_hi);
                        if (p.causal) lane_need = lane_need || (COL ? pos_a + 8 > other * kTile : other * kTile + kTile - 1 > pos_a);
                        if (COL) {
                            lane_need = lane_need || pad_a || pad_b;
                        } else if (kpm_row != nullptr) {
                            const uint8_t* kb = kpm_row + other * kTile;
                            if (__any_sync(0xffffffffu, (kb[lane] | kb[32 + lane]) != 0)) {
#pragma unroll
                                for (int i = 0; i < 16; ++i)
                                    padbits |= (kpm_row[other0 + 8 * (i >> 1) + (i & 1)] != 0 ? 1u : 0u) << i;
                                lane_need = lane_need || padbits != 0u;
                            }
                        }
                        need = __any_sync(0xffffffffu, lane_need) != 0;
                    }
                    auto emit = [&](auto masked_tag) {
                        constexpr bool M = decltype(masked_tag)::value;
#pragma unroll
                        for (int u = 0; u < 8; ++u) {
                            float pa[2], pb[2], da[2], db[2];
#pragma unroll
                            for (int e = 0; e < 2; ++e) {
                                float lse_a, lse_b, dl_a, dl_b;
                                if (COL) {
                                    lse_a = lse_b = e == 0 ? cs[u].x : cs[u].z;
                                    dl_a = dl_b = e == 0 ? cs[u].y : cs[u].w;
                                } else {
                                    lse_a = st_a.x; dl_a = st_a.y; lse_b = st_b.x; dl_b = st_b.y;
                                }
                                pa[e] = attn_exp2(fmaf(__uint_as_float(r1[4 * u + e]), c2, -lse_a));
                                pb[e] = attn_exp2(fmaf(__uint_as_float(r1[4 * u + 2 + e]), c2, -lse_b));
                                if (M) {
                                    const int opos = other0 + 8 * u + e;
                                    bool m_a, m_b;
                                    if (COL) {
                                        // lane rows are keys, columns are queries
                                        m_a = pad_a || (p.causal && pos_a > opos);
                                        m_b = pad_b || (p.causal && pos_a + 8 > opos);
                                    } else {
                                        const bool pad = ((padbits >> (2 * u + e)) & 1u) != 0;
                                        m_a = pad || (p.causal && opos > pos_a);
                                        m_b = pad || (p.causal && opos > pos_a + 8);
                                    }
                                    if (!(u < 4 ? sub_lo : sub_hi)) { m_a = true; m_b = true; }
                                    if (m_a) pa[e] = 0.f;
                                    if (m_b) pb[e] = 0.f;
                                }
                                da[e] = pa[e] * (__uint_as_float(r2[4 * u + e]) - dl_a) * sc;
                                db[e] = pb[e] * (__uint_as_float(r2[4 * u + 2 + e]) - dl_b) * sc;
                            }
                            const uint32_t addr = tile0 + (((uint32_t)u ^ op_xor) << 4);
                            if (COL) {
                                // tile 0: P^T, tile 1: dS^T
                                asm volatile("st.shared.b32 [%0], %1;" ::"r"(addr), "r"(pack2<BF16>(pa[0], pa[1])) : "memory");
                                asm volatile("st.shared.b32 [%0], %1;" ::"r"(addr + 8 * 128), "r"(pack2<BF16>(pb[0], pb[1])) : "memory");
                                asm volatile("st.shared.b32 [%0], %1;" ::"r"(addr + kTileBytes), "r"(pack2<BF16>(da[0], da[1])) : "memory");
                                asm volatile("st.shared.b32 [%0], %1;" ::"r"(addr + kTileBytes + 8 * 128), "r"(pack2<BF16>(db[0], db[1])) : "memory");
                            } else {
                                asm volatile("st.shared.b32 [%0], %1;" ::"r"(addr), "r"(pack2<BF16>(da[0], da[1])) : "memory");
                                asm volatile("st.shared.b32 [%0], %1;" ::"r"(addr + 8 * 128), "r"(pack2<BF16>(db[0], db[1])) : "memory");
                            }
                        }
                    };
                    if (MASKED && need) emit(std::true_type{});
                    else                emit(std::false_type{});
                    fence_async_shared();           // generic-proxy writes -> visible to the tensor core's reads
                    __syncwarp();
                    if (lane == 0) mbar_arrive(&bars->op_full[ob]);
                }
                s_no += n;
                if (!ok) break;
                // The groups store the accumulators of alternate items.  The rule must not depend on the
                // data: an mbarrier parity wait tells the current phase from the one before only, so
                // o_full / o_empty of the items of one parity are always waited on by the same group, in
                // every phase.  (Letting the owner of an item's last block store it was 3 % faster and
                // wrong: with rows of 1-3 blocks and several items per CTA a group skipped phases, passed
                // a wait one phase early and the kernel ended in a time-out.)
                if (wg == (o_no & 1)) {
                    const int ob_acc = o_no & (p.obufs - 1);
                    ok = __all_sync(0xffffffffu, mbar_wait(&bars->o_full[o_no & 1], (uint32_t)(o_no >> 1) & 1u, abort_flag, p.status)) != 0;
                    if (!ok) break;
                    tc_fence_after();
#pragma unroll
                    for (int a = 0; a < kOuts; ++a) {
                        uint16_t* out = a == 0 ? p.out0 : p.out1;
                        for (int c = 0; c < p.head_dim; c += 32) {
                            uint32_t r0[16];
                            const uint32_t acc0 = tmem_base + lane_field + (uint32_t)(kBwdAccCol0 + (ob_acc * kOuts + a) * p.parts * p.head_dim + c);
                            tc_ld_16x256b_x4(acc0, r0);
                            tc_wait_ld();
                            for (int q = 1; q < p.parts; ++q) {          // add the other partial accumulators
                                uint32_t rq[16];
                                tc_ld_16x256b_x4(acc0 + (uint32_t)(q * p.head_dim), rq);
                                tc_wait_ld();
#pragma unroll
                                for (int i = 0; i < 16; ++i) r0[i] = __float_as_uint(__uint_as_float(r0[i]) + __uint_as_float(rq[i]));
                            }
                            if (a == kOuts - 1 && c + 32 >= p.head_dim) release_accumulator(&bars->o_empty[o_no & 1], lane);
                            uint32_t ta[4], tb2[4];
#pragma unroll
                            for (int u = 0; u < 4; ++u) {
                                ta[u] = pack2<BF16>(__uint_as_float(r0[4 * u]), __uint_as_float(r0[4 * u + 1]));
                                tb2[u] = pack2<BF16>(__uint_as_float(r0[4 * u + 2]), __uint_as_float(r0[4 * u + 3]));
                            }
                            quad_transpose(ta, q4);          // now columns c + 8 * q4 .. + 7 of the row
                            quad_transpose(tb2, q4);
                            *reinterpret_cast<uint4*>(out + out_a + c + 8 * q4) = make_uint4(ta[0], ta[1], ta[2], ta[3]);
                            *reinterpret_cast<uint4*>(out + out_b + c + 8 * q4) = make_uint4(tb2[0], tb2[1], tb2[2], tb2[3]);
                        }
                    }
                }
                ++o_no;
            }
            pre = pre_next;
            cur.advance();
        }
    }

    // ---------------------------------------------------------------- teardown
    tc_fence_before();
    __syncthreads();
    if (warp == kBwdProducerWarp) {
        __syncwarp();
        tc_fence_after();
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"((uint32_t)kBwdTmemCols)
                     : "memory");
    }
}

}  // namespace

namespace {

#include "bsa_attention_bwd_rows.cuh"

// dQ by block rows with head dim 64: the two-pipeline kernel.
int launch_backward_rows_pipes(int dtype, bool masked, const CUtensorMap& q, const CUtensorMap& dout, const CUtensorMap& k,
                               const CUtensorMap& v, BwdParams p, cudaStream_t stream) {
    using KernelFn = void (*)(const CUtensorMap, const CUtensorMap, const CUtensorMap, const CUtensorMap, const BwdParams);
    KernelFn kernel;
    if (dtype == BSA_DTYPE_BF16) kernel = masked ? attention_backward_rows_pipes_kernel<true, true> : attention_backward_rows_pipes_kernel<true, false>;
    else                         kernel = masked ? attention_backward_rows_pipes_kernel<false, true> : attention_backward_rows_pipes_kernel<false, false>;
    // at least 80 KB, so that never more than two CTAs (256 TMEM columns each) share an SM
    int smem_bytes = 1024 + 2 * kBwdRowTiles * kTileBytes + (int)sizeof(BwdRowBarriers);
    if (smem_bytes < 80 * 1024) smem_bytes = 80 * 1024;
    if (!ensure_dynamic_smem(reinterpret_cast<const void*>(kernel), smem_bytes)) return BSA_ERR_LAUNCH;
    const int sms = sm_count();
    if (sms <= 0) return BSA_ERR_LAUNCH;
    // walkers of the work-item list: the two pipelines of every CTA
    const int wanted = (p.items + 1) / 2;
    const unsigned grid = (unsigned)(wanted < 2 * sms ? wanted : 2 * sms);
    p.stride_z = 2 * (int)grid / p.groups;
    p.stride_rem = 2 * (int)grid % p.groups;
    kernel<<<grid, 12 * 32, smem_bytes, stream>>>(q, dout, k, v, p);
    return launch_status();
}

#include "bsa_attention_bwd_cols.cuh"

// dK, dV by block columns with head dim 64: the two-pipeline kernel (one CTA per SM).
int launch_backward_cols_pipes(int dtype, bool masked, const CUtensorMap& k, const CUtensorMap& v, const CUtensorMap& q,
                               const CUtensorMap& dout, BwdParams p, cudaStream_t stream) {
    using KernelFn = void (*)(const CUtensorMap, const CUtensorMap, const CUtensorMap, const CUtensorMap, const BwdParams);
    KernelFn kernel;
    if (dtype == BSA_DTYPE_BF16) kernel = masked ? attention_backward_cols_pipes_kernel<true, true> : attention_backward_cols_pipes_kernel<true, false>;
    else                         kernel = masked ? attention_backward_cols_pipes_kernel<false, true> : attention_backward_cols_pipes_kernel<false, false>;
    const int smem_bytes = 1024 + 2 * kBwdColTiles * kTileBytes + 2 * kBwdColRing * kBwdStatBytes + (int)sizeof(BwdColBarriers);
    if (!ensure_dynamic_smem(reinterpret_cast<const void*>(kernel), smem_bytes)) return BSA_ERR_LAUNCH;
    const int sms = sm_count();
    if (sms <= 0) return BSA_ERR_LAUNCH;
    // walkers of the work-item list: the two pipelines of every CTA
    const int wanted = (p.items + 1) / 2;
    const unsigned grid = (unsigned)(wanted < sms ? wanted : sms);
    p.stride_z = 2 * (int)grid / p.groups;
    p.stride_rem = 2 * (int)grid % p.groups;
    kernel<<<grid, kBwdColWarps * 32, smem_bytes, stream>>>(k, v, q, dout, p);
    return launch_status();
}

// One launch of the backward kernel template (by rows or by columns).
template <bool COL>
int launch_backward(int dtype, bool masked, const CUtensorMap& x1, const CUtensorMap& x2, const CUtensorMap& y1,
                    const CUtensorMap& y2, BwdParams p, cudaStream_t stream) {
    using KernelFn = void (*)(const CUtensorMap, const CUtensorMap, const CUtensorMap, const CUtensorMap, const BwdParams);
    KernelFn kernel;
    if (dtype == BSA_DTYPE_BF16) kernel = masked ? attention_backward_kernel<COL, true, true> : attention_backward_kernel<COL, true, false>;
    else                         kernel = masked ? attention_backward_kernel<COL, false, true> : attention_backward_kernel<COL, false, false>;
    // Shared memory (227 KB): head dim 64: two X pairs (32 KB), 8 (by rows) or 4 (by columns) Y stages of
    // 16 KB, 4 operand buffers of 8 / 16 KB; head dim 128: one X pair (32 KB), 4 Y stages of 32 KB,
    // 4 operand buffers of 8 KB by rows, 2 of 16 KB by columns.
    p.xbufs = p.dtiles == 1 ? 2 : 1;
    p.ring = (p.dtiles == 1 && !COL) ? 8 : 4;
    p.ring_shift = p.ring == 8 ? 3 : 2;
    // The 256 TMEM columns beside the T buffers: two accumulator sets where they fit (the next item
    // accumulates while an item is stored); by rows with head dim 64 also two partial accumulators fed
    // by two issuers.  (Partial accumulators fed by one issuer were measured to gain nothing: chained
    // MMAs into one accumulator are not what bounds the kernel.)
    p.obufs = (COL && p.dtiles == 2) ? 1 : 2;
    p.parts = (!COL && p.dtiles == 1) ? 2 : 1;
    p.out_issuers = COL ? 2 : p.parts;
    p.opbufs = (COL && p.dtiles == 2) ? 2 : 4;
    p.op_shift = p.opbufs == 4 ? 2 : 1;
    int smem_bytes = 1024 + ((p.xbufs * 2 + p.ring * 2) * p.dtiles + p.opbufs * (COL ? 2 : 1)) * kTileBytes +
                     (COL ? p.ring * kBwdStatBytes : 0) + (int)sizeof(BwdBarriers);
    // more than half of an SM's shared memory: the CTA allocates all 512 TMEM columns and must be alone
    if (smem_bytes < 116 * 1024) smem_bytes = 116 * 1024;
    if (!ensure_dynamic_smem(reinterpret_cast<const void*>(kernel), smem_bytes)) return BSA_ERR_LAUNCH;
    const int sms = sm_count();
    if (sms <= 0) return BSA_ERR_LAUNCH;
    const unsigned grid = (unsigned)(p.items < sms ? p.items : sms);
    p.stride_z = (int)grid / p.groups;
    p.stride_rem = (int)grid % p.groups;
    kernel<<<grid, bwd_warps<COL>() * 32, smem_bytes, stream>>>(x1, x2, y1, y2, p);
    return launch_status();
}

}  // namespace

// Host side of bsa_attention_backward (arguments already validated by the caller).
int attention_backward(int dtype, const void* q, const void* k, const void* v, const void* o, const void* dout,
                       const float* lse, void* dq, void* dk, void* dv,
                       const int32_t* row_blocks, const int32_t* row_table,
                       const int32_t* col_blocks, const int32_t* col_table,
                       int64_t nnz, int64_t block_rows, int64_t block_cols, int64_t batches, int64_t head_dim,
                       float scale, int causal, const uint8_t* kpm, int64_t kpm_batches, int64_t kpm_stride,
                       int quadrants, float2* stats, uint32_t* workspace, cudaStream_t stream) {
    const int64_t seq_q = block_rows * kTile, seq_k = block_cols * kTile;
    const long long rows = (long long)batches * seq_q;
    if (head_dim != kTile) {        // head dim 64: the kernel by rows computes the statistics itself
        const int lanes = (int)head_dim / 8;
        const long long threads = rows * lanes;
        const unsigned grid = (unsigned)((threads + 255) / 256);
        if (dtype == BSA_DTYPE_BF16)
            attention_backward_stats_kernel<true><<<grid, 256, 0, stream>>>(
                static_cast<const uint16_t*>(o), static_cast<const uint16_t*>(dout), lse, stats, rows, (int)head_dim);
        else
            attention_backward_stats_kernel<false><<<grid, 256, 0, stream>>>(
                static_cast<const uint16_t*>(o), static_cast<const uint16_t*>(dout), lse, stats, rows, (int)head_dim);
        const int st = launch_status();
        if (st != BSA_OK) return st;
    }
    CUtensorMap map_q, map_k, map_v, map_do;
    bool ok = make_map(&map_q, dtype, q, batches, seq_q, head_dim);
    ok &= make_map(&map_do, dtype, dout, batches, seq_q, head_dim);
    ok &= make_map(&map_k, dtype, k, batches, seq_k, head_dim);
    ok &= make_map(&map_v, dtype, v, batches, seq_k, head_dim);
    if (!ok) return BSA_ERR_DRIVER;

    BwdParams p{};
    p.status = workspace;
    p.nnz = (int)nnz; p.batches = (int)batches;
    p.chunks = 1;
    p.seq_q = (int)seq_q; p.seq_k = (int)seq_k; p.head_dim = (int)head_dim;
    p.dtiles = (int)(head_dim / kTile);
    p.scale = scale;
    p.scale_log2 = scale * kLog2e;
    p.causal = causal;
    p.quadrants = quadrants;
    p.kpm = kpm;
    p.kpm_div = kpm ? (int)(batches / kpm_batches) : 1;
    p.kpm_stride = kpm_stride;
    p.stats = stats;
    p.stats_out = stats;
    p.o = static_cast<const uint16_t*>(o);
    p.dout = static_cast<const uint16_t*>(dout);
    p.lse = lse;
    // instruction descriptors: fp32 accumulate, fp16 / bf16 operands, M = 64; T: both operands K-major,
    // N = 64; accumulations: B (a Y tile set) with N contiguous, N = head_dim
    const uint32_t fmt = dtype == BSA_DTYPE_BF16 ? 1u : 0u;
    const uint32_t common = (1u << 4) | (fmt << 7) | (fmt << 10) | ((uint32_t)(kTile >> 4) << 24);
    p.idesc_t = common | ((uint32_t)(kTile >> 3) << 17);
    p.idesc_acc = common | (1u << 16) | ((uint32_t)(head_dim >> 3) << 17);
    const bool masked = causal != 0 || kpm != nullptr || quadrants != 0;

    // dQ by rows: X = (Q_r, dO_r), Y = (K_c, V_c)
    p.blocks = reinterpret_cast<const BlockDesc*>(row_blocks);
    p.table = row_table;
    p.groups = (int)block_rows;
    p.items = (int)(batches * block_rows);
    p.out0 = static_cast<uint16_t*>(dq);
    p.out1 = nullptr;
    int st = BSA_OK;
    st = head_dim == kTile ? launch_backward_rows_pipes(dtype, masked, map_q, map_do, map_k, map_v, p, stream)
                           : launch_backward<false>(dtype, masked, map_q, map_do, map_k, map_v, p, stream);
    if (st != BSA_OK) return st;
    // dV, dK by columns: X = (K_c, V_c), Y = (Q_r, dO_r)
    p.blocks = reinterpret_cast<const BlockDesc*>(col_blocks);
    p.table = col_table;
    p.groups = (int)block_cols;
    p.items = (int)(batches * block_cols);
    p.out0 = static_cast<uint16_t*>(dv);
    p.out1 = static_cast<uint16_t*>(dk);
    return head_dim == kTile ? launch_backward_cols_pipes(dtype, masked, map_k, map_v, map_q, map_do, p, stream)
                             : launch_backward<true>(dtype, masked, map_k, map_v, map_q, map_do, p, stream);
}

}  // namespace bsa

extern "C" int bsa_attention_backward(int dtype, const void* q, const void* k, const void* v, const void* o,
                                      const void* dout, const float* lse, void* dq, void* dk, void* dv,
                                      const int32_t* row_blocks, const int32_t* row_table,
                                      const int32_t* col_blocks, const int32_t* col_table,
                                      int64_t nnz, int64_t block_rows, int64_t block_cols, int64_t batches,
                                      int64_t head_dim, int block, float scale, int causal,
                                      const uint8_t* key_padding_mask, int64_t kpm_batches, int64_t kpm_stride,
                                      int quadrant_masks, void* stats, size_t stats_bytes,
                                      void* workspace, size_t workspace_bytes, void* stream) {
    using namespace bsa;
    if (dtype != BSA_DTYPE_F32 && dtype != BSA_DTYPE_F16 && dtype != BSA_DTYPE_BF16) return BSA_ERR_BAD_DTYPE;
    if (!valid_block(block)) return BSA_ERR_BAD_BLOCK;
    if (!q || !k || !v || !o || !dout || !lse || !dq || !dk || !dv || !row_blocks || !row_table || !col_blocks || !col_table)
        return BSA_ERR_NULL_POINTER;
    if (!workspace || workspace_bytes < BSA_WORKSPACE_BYTES) return BSA_ERR_WORKSPACE;
    if (nnz < 0 || block_rows <= 0 || block_cols <= 0 || batches < 0 || head_dim <= 0) return BSA_ERR_BAD_SHAPE;
    if (block_rows > 65535 || block_cols > 65535 || nnz > block_rows * block_cols) return BSA_ERR_BAD_SHAPE;
    if (!attention_supports(dtype, head_dim, block)) return dtype == BSA_DTYPE_F32 ? BSA_ERR_BAD_DTYPE : BSA_ERR_BAD_SHAPE;
    if (batches > 65535 || batches * block_rows >= ((int64_t)1 << 30) || batches * block_cols >= ((int64_t)1 << 30) ||
        block_rows * block >= ((int64_t)1 << 31) || block_cols * block >= ((int64_t)1 << 31))
        return BSA_ERR_TOO_LARGE;
    if (!stats || stats_bytes < (size_t)batches * block_rows * block * 8) return BSA_ERR_WORKSPACE;
    if (!aligned16(q) || !aligned16(k) || !aligned16(v) || !aligned16(o) || !aligned16(dout) || !aligned16(dq) ||
        !aligned16(dk) || !aligned16(dv) || !aligned16(stats))
        return BSA_ERR_ALIGNMENT;
    if (key_padding_mask && (kpm_batches <= 0 || batches % kpm_batches != 0 || kpm_stride < block_cols * block))
        return BSA_ERR_BAD_SHAPE;
    if (batches == 0) return BSA_OK;
    return attention_backward(dtype, q, k, v, o, dout, lse, dq, dk, dv, row_blocks, row_table, col_blocks, col_table,
                              nnz, block_rows, block_cols, batches, head_dim, scale, causal, key_padding_mask,
                              kpm_batches, kpm_stride, quadrant_masks != 0, static_cast<float2*>(stats),
                              static_cast<uint32_t*>(workspace), static_cast<cudaStream_t>(stream));
}
