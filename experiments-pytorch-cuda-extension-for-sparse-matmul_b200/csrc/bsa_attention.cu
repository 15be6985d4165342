// Fused block-sparse attention forward (sm_100a only):
//   O = softmax_rows(scale * Q K^T + masks, restricted to the layout) V
// in one kernel, so the score and probability blocks never travel through HBM.  The reference
// composes this from three launches of its matmul and softmax kernels (sdd: sparse_smm_gpu.cu:22-99,
// softmax: sparse_softmax.cu:113-155, dsd: sparse_smm_gpu.cu:101-183), each writing the
// [batch, nnz, block, block] tensor to memory; this entry point has no counterpart there and
// exists beside the three unfused operators.
//
// Work item = one block row r of one batch entry (64 query rows).  Two passes over the row's
// blocks c_0 .. c_{n-1}, both on the tensor cores (tcgen05, fp32 accumulators in TMEM):
//   pass 1   S_j = Q_r K_{c_j}^T              -> row maxima m of scale * S (+ masks)
//   pass 2   S_j again, P_j = exp(scale * S_j - m) written as a 16-bit K-major operand tile to
//            shared memory, O += P_j V_{c_j}   -> row sums l accumulate next to it
//   end      O / l -> global, lse = m + log l
// Recomputing S costs tensor-core time that is idle anyway and removes the running-maximum
// rescaling of O (and its dependency chain between softmax and the second matmul) that a
// one-pass online softmax needs.  K tiles are read twice, the second time from L2.
//
// A CTA has 6 warps and 256 TMEM columns, two CTAs share an SM and overlap each other's
// prologues and epilogues:
//   warp 0     TMA producer: Q once per item, K tiles (pass 1), K and V tiles (pass 2)
//   warp 1     tcgen05.mma issuer; S is double buffered so Q K^T of block j + 1 runs while the
//              softmax warps work on block j
//   warps 2-5  softmax: tcgen05.ld with the 16x256b shape (every lane owns 2 rows x 16 columns
//              of a 64 x 64 block), masks, max / exp / sum, pack, 4x4 quad transposes, swizzled
//              128-bit shared-memory stores of P; at the end the same for O to global memory.
// All waits are bounded (BSA_ERR_DEVICE_TIMEOUT in the workspace word).
#include "bsa_tc_common.cuh"

namespace bsa {
namespace {

constexpr int kAttnWarps = 6;
constexpr int kAttnThreads = kAttnWarps * 32;
constexpr int kAttnTmemCols = 256;      // O: columns 0 .. head_dim - 1; S buffers: 128 .. 191, 192 .. 255
constexpr int kSCol0 = 128;
constexpr int kMaxRing = 4;

struct __align__(8) AttnBarriers {
    uint64_t q_full, q_empty;
    uint64_t k_full[kMaxRing], k_empty[kMaxRing];
    uint64_t v_full[kMaxRing], v_empty[kMaxRing];
    uint64_t s_full[2], s_empty[2];
    uint64_t p_full[2], p_empty[2];
    uint64_t o_full, o_empty;
    uint64_t drain;
    uint32_t tmem_base;
    int abort_flag;
};

struct AttnParams {
    const BlockDesc* blocks;   // row layout
    const int32_t* table;
    uint32_t* status;          // workspace word
    int nnz, groups, batches;  // groups = block rows
    int chunks, items;         // chunks = 1 (kept for the shared cursor)
    int stride_z, stride_rem;
    int seq_q, seq_k, head_dim;
    int dtiles;                // head_dim / 64
    int ring, ring_shift;      // K and V pipeline depth (a power of two) and its log2
    float scale_log2;          // scale * log2(e)
    int causal;
    const uint8_t* kpm;        // key padding mask or nullptr
    int kpm_div;               // batch entries per mask row
    long long kpm_stride;
    uint16_t* o;
    float* lse;
    uint32_t idesc_qk, idesc_pv;
};

__device__ __forceinline__ float attn_exp2(float x) {
    float y;
    asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
    return y;
}

template <bool BF16>
__device__ __forceinline__ uint32_t pack2(float lo, float hi) {
    if (BF16) {
        __nv_bfloat162 h = __floats2bfloat162_rn(lo, hi);
        return *reinterpret_cast<uint32_t*>(&h);
    }
    __half2 h = __floats2half2_rn(lo, hi);
    return *reinterpret_cast<uint32_t*>(&h);
}

template <bool BF16>
__global__ void __launch_bounds__(kAttnThreads, 2)
attention_forward_kernel(const __grid_constant__ CUtensorMap map_q, const __grid_constant__ CUtensorMap map_k,
                         const __grid_constant__ CUtensorMap map_v, const AttnParams p) {
    extern __shared__ uint8_t smem_raw[];
    uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~(uintptr_t)1023);
    // tiles: Q (dtiles), K ring (ring x dtiles), V ring (ring x dtiles), P (2)
    const int set_bytes = p.dtiles * kTileBytes;            // one Q / K / V tile set
    uint8_t* q_smem = smem;
    uint8_t* k_smem = q_smem + set_bytes;
    uint8_t* v_smem = k_smem + p.ring * set_bytes;
    uint8_t* p_smem = v_smem + p.ring * set_bytes;
    AttnBarriers* bars = reinterpret_cast<AttnBarriers*>(p_smem + 2 * kTileBytes);
    int* abort_flag = &bars->abort_flag;

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int ring_mask = p.ring - 1;

    if (threadIdx.x == 0) {
        mbar_init(&bars->q_full, 1); mbar_init(&bars->q_empty, 1);
        for (int s = 0; s < kMaxRing; ++s) {
            mbar_init(&bars->k_full[s], 1); mbar_init(&bars->k_empty[s], 1);
            mbar_init(&bars->v_full[s], 1); mbar_init(&bars->v_empty[s], 1);
        }
        for (int s = 0; s < 2; ++s) {
            mbar_init(&bars->s_full[s], 1); mbar_init(&bars->s_empty[s], 4);
            mbar_init(&bars->p_full[s], 4); mbar_init(&bars->p_empty[s], 1);
        }
        mbar_init(&bars->o_full, 1); mbar_init(&bars->o_empty, 4);
        mbar_init(&bars->drain, 1);
        bars->abort_flag = 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
        fence_async_shared();
    }
    if (warp == 1) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;"
                     ::"r"(smem_u32(&bars->tmem_base)), "r"((uint32_t)kAttnTmemCols) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem_base = *(volatile uint32_t*)&bars->tmem_base;

    if (warp == 0) {
        // ------------------------------------------------------------ TMA producer
        int k_no = 0, v_no = 0, q_no = 0;          // tile sets loaded so far
        bool ok = true;
        Cursor cur;
        cur.init(p);
        BlockDesc pre = cur.valid() ? load_first_chunk(p.blocks, cur.first, cur.count, lane) : BlockDesc{0, 0};
        while (ok && cur.valid()) {
            BlockDesc pre_next{0, 0};
            if (cur.has_next()) pre_next = load_first_chunk(p.blocks, cur.next_first(), cur.next_count(), lane);
            const int n = cur.count;
            if (n > 0) {
                if (lane == 0) {
                    ok = mbar_wait(&bars->q_empty, (uint32_t)(q_no & 1) ^ 1u, abort_flag, p.status);
                    if (ok) {
                        mbar_expect_tx(&bars->q_full, (uint32_t)set_bytes);
                        for (int t = 0; t < p.dtiles; ++t)
                            tma_load_3d(q_smem + t * kTileBytes, &map_q, &bars->q_full, t * kTile, cur.g * kTile, cur.z);
                    }
                }
                ++q_no;
                ok = __shfl_sync(0xffffffffu, (int)ok, 0) != 0;
                for (int pass = 0; ok && pass < 2; ++pass) {
                    DescWindow win;                 // indices must not decrease: one window per pass
                    win.begin(p.blocks, cur.first, cur.count, pre, lane);
                    for (int j = 0; ok && j < n; ++j) {
                        const int col = win.get(p.blocks, cur.first, cur.count, j, lane).col();
                        if (lane == 0) {
                            const int ks = k_no & ring_mask;
                            ok = mbar_wait(&bars->k_empty[ks], ((uint32_t)(k_no >> p.ring_shift) & 1u) ^ 1u, abort_flag, p.status);
                            if (ok) {
                                mbar_expect_tx(&bars->k_full[ks], (uint32_t)set_bytes);
                                for (int t = 0; t < p.dtiles; ++t)
                                    tma_load_3d(k_smem + ks * set_bytes + t * kTileBytes, &map_k, &bars->k_full[ks],
                                                t * kTile, col * kTile, cur.z);
                            }
                            if (ok && pass == 1) {
                                const int vs = v_no & ring_mask;
                                ok = mbar_wait(&bars->v_empty[vs], ((uint32_t)(v_no >> p.ring_shift) & 1u) ^ 1u, abort_flag, p.status);
                                if (ok) {
                                    mbar_expect_tx(&bars->v_full[vs], (uint32_t)set_bytes);
                                    for (int t = 0; t < p.dtiles; ++t)
                                        tma_load_3d(v_smem + vs * set_bytes + t * kTileBytes, &map_v, &bars->v_full[vs],
                                                    t * kTile, col * kTile, cur.z);
                                }
                            }
                        }
                        ++k_no;
                        if (pass == 1) ++v_no;
                        ok = __shfl_sync(0xffffffffu, (int)ok, 0) != 0;
                    }
                }
            }
            pre = pre_next;
            cur.advance();
        }
        if (lane == 0 && *(volatile int*)abort_flag) {
            // Give copies that were issued a bounded chance to land before the CTA exits.
            const unsigned long long t0 = global_ns();
            for (int s = 0; s < p.ring; ++s) {
                while (!mbar_try_wait(&bars->k_full[s], 0) && !mbar_try_wait(&bars->k_full[s], 1) &&
                       global_ns() - t0 < kWaitLimitNs / 4) {}
                while (!mbar_try_wait(&bars->v_full[s], 0) && !mbar_try_wait(&bars->v_full[s], 1) &&
                       global_ns() - t0 < kWaitLimitNs / 4) {}
            }
            while (!mbar_try_wait(&bars->q_full, 0) && !mbar_try_wait(&bars->q_full, 1) &&
                   global_ns() - t0 < kWaitLimitNs / 4) {}
        }
        __syncwarp();
    } else if (warp == 1) {
        // ------------------------------------------------------------ MMA issuer
        if (lane == 0) {
            int k_no = 0, v_no = 0, s_no = 0, p_no = 0, q_no = 0;   // consumed K / V sets, produced S, consumed P, items
            bool ok = true;
            const uint32_t idesc_qk = p.idesc_qk, idesc_pv = p.idesc_pv;
            // S_j = Q K_{c_j}^T into S buffer s_no & 1
            auto issue_qk = [&]() -> bool {
                const int ks = k_no & ring_mask, sb = s_no & 1;
                if (!mbar_wait(&bars->k_full[ks], (uint32_t)(k_no >> p.ring_shift) & 1u, abort_flag, p.status)) return false;
                if (!mbar_wait(&bars->s_empty[sb], ((uint32_t)(s_no >> 1) & 1u) ^ 1u, abort_flag, p.status)) return false;
                tc_fence_after();
                const uint32_t d = tmem_base + (uint32_t)(kSCol0 + sb * kTile);
                for (int t = 0; t < p.dtiles; ++t) {
                    const uint64_t da = make_tile_desc(smem_u32(q_smem + t * kTileBytes), false);
                    const uint64_t db = make_tile_desc(smem_u32(k_smem + ks * set_bytes + t * kTileBytes), false);
#pragma unroll
                    for (int kk = 0; kk < kTile / 16; ++kk)
                        tc_mma_f16(d, da + (uint64_t)(kk * 2), db + (uint64_t)(kk * 2), idesc_qk, (t > 0 || kk > 0) ? 1u : 0u);
                }
                tc_commit(&bars->k_empty[ks]);
                tc_commit(&bars->s_full[sb]);
                ++k_no; ++s_no;
                return true;
            };
            Cursor cur;
            cur.init(p);
            for (; ok && cur.valid(); cur.advance()) {
                const int n = cur.count;
                if (n == 0) continue;               // empty row: the softmax warps write zeros on their own
                ok = mbar_wait(&bars->q_full, (uint32_t)(q_no & 1), abort_flag, p.status);
                if (!ok) break;
                for (int j = 0; ok && j < n; ++j) ok = issue_qk();          // pass 1
                if (ok) ok = issue_qk();                                    // pass 2, block 0
                for (int j = 0; ok && j < n; ++j) {
                    if (j + 1 < n) {
                        ok = issue_qk();            // runs while the softmax warps work on block j
                        if (!ok) break;
                    } else {
                        tc_commit(&bars->q_empty);  // last read of Q has been issued
                    }
                    const int vs = v_no & ring_mask, pb = p_no & 1;
                    if (j == 0) ok = mbar_wait(&bars->o_empty, (uint32_t)(q_no & 1) ^ 1u, abort_flag, p.status);
                    if (ok) ok = mbar_wait(&bars->v_full[vs], (uint32_t)(v_no >> p.ring_shift) & 1u, abort_flag, p.status);
                    if (ok) ok = mbar_wait(&bars->p_full[pb], (uint32_t)(p_no >> 1) & 1u, abort_flag, p.status);
                    if (!ok) break;
                    tc_fence_after();
                    // O += P_j V_{c_j}: A = P (K-major), B = V tiles (N contiguous), N = head_dim
                    const uint64_t da = make_tile_desc(smem_u32(p_smem + pb * kTileBytes), false);
                    const uint64_t db = make_tile_desc(smem_u32(v_smem + vs * set_bytes), true);
#pragma unroll
                    for (int kk = 0; kk < kTile / 16; ++kk)
                        tc_mma_f16(tmem_base, da + (uint64_t)(kk * 2), db + (uint64_t)(kk * (2048 >> 4)), idesc_pv,
                                   (j > 0 || kk > 0) ? 1u : 0u);
                    tc_commit(&bars->v_empty[vs]);
                    tc_commit(&bars->p_empty[pb]);
                    if (j == n - 1) tc_commit(&bars->o_full);
                    ++v_no; ++p_no;
                }
                ++q_no;
            }
            // All MMAs issued by this thread must have retired before TMEM is freed.
            tc_commit(&bars->drain);
            mbar_wait(&bars->drain, 0, abort_flag, p.status);
        }
        __syncwarp();
    } else {
        // ------------------------------------------------------------ softmax warps
        const int quad = warp & 3;                  // TMEM sub-partition this warp may read
        const int q4 = lane & 3;                    // position in the quad: columns 8u + 2 * q4 + {0, 1}
        const int row_a = quad * 16 + (lane >> 2);  // this lane's two rows of the 64-row block
        const int row_b = row_a + 8;
        const uint32_t lane_field = (uint32_t)(quad * 32) << 16;
        const bool masked_op = p.causal != 0 || p.kpm != nullptr;
        int s_no = 0, p_no = 0, o_no = 0;
        bool ok = true;
        Cursor cur;
        cur.init(p);
        BlockDesc pre = cur.valid() ? load_first_chunk(p.blocks, cur.first, cur.count, lane) : BlockDesc{0, 0};
        while (ok && cur.valid()) {
            BlockDesc pre_next{0, 0};
            if (cur.has_next()) pre_next = load_first_chunk(p.blocks, cur.next_first(), cur.next_count(), lane);
            const int n = cur.count;
            const size_t o_row_a = ((size_t)cur.z * p.seq_q + (size_t)cur.g * kTile + row_a) * p.head_dim;
            const size_t o_row_b = o_row_a + (size_t)8 * p.head_dim;
            const size_t lse_a = (size_t)cur.z * p.seq_q + (size_t)cur.g * kTile + row_a;
            if (n == 0) {
                // a block row without blocks: zeros, lse = -inf
                for (int c = q4 * 8; c < p.head_dim; c += 32) {
                    *reinterpret_cast<uint4*>(p.o + o_row_a + c) = make_uint4(0u, 0u, 0u, 0u);
                    *reinterpret_cast<uint4*>(p.o + o_row_b + c) = make_uint4(0u, 0u, 0u, 0u);
                }
                if (q4 == 0 && p.lse) { p.lse[lse_a] = -INFINITY; p.lse[lse_a + 8] = -INFINITY; }
            } else {
                const uint8_t* kpm_row = p.kpm ? p.kpm + (size_t)(cur.z / p.kpm_div) * p.kpm_stride : nullptr;
                const int qpos_a = cur.g * kTile + row_a;
                // Bits 0-15: columns (u, e) of row a that are masked in block `col`; bits 16-31: row b.
                auto block_mask = [&](int col) -> uint32_t {
                    uint32_t m = 0;
                    const int k0 = col * kTile + 2 * q4;
                    if (p.causal && col * kTile + kTile - 1 > qpos_a) {
#pragma unroll
                        for (int u = 0; u < 8; ++u)
#pragma unroll
                            for (int e = 0; e < 2; ++e) {
                                const int kpos = k0 + 8 * u + e;
                                if (kpos > qpos_a) m |= 1u << (2 * u + e);
                                if (kpos > qpos_a + 8) m |= 1u << (16 + 2 * u + e);
                            }
                    }
                    if (kpm_row) {
#pragma unroll
                        for (int u = 0; u < 8; ++u) {
                            if (kpm_row[k0 + 8 * u]) m |= 0x00010001u << (2 * u);
                            if (kpm_row[k0 + 8 * u + 1]) m |= 0x00010001u << (2 * u + 1);
                        }
                    }
                    return m;
                };
                const float c2 = p.scale_log2;
                // ---- pass 1: row maxima of scale * log2(e) * S
                float m_a = -INFINITY, m_b = -INFINITY;
                DescWindow win;
                win.begin(p.blocks, cur.first, cur.count, pre, lane);
                for (int j = 0; ok && j < n; ++j, ++s_no) {
                    const int sb = s_no & 1;
                    const int col = masked_op ? win.get(p.blocks, cur.first, cur.count, j, lane).col() : 0;
                    const uint32_t mask = masked_op ? block_mask(col) : 0u;
                    ok = __all_sync(0xffffffffu, mbar_wait(&bars->s_full[sb], (uint32_t)(s_no >> 1) & 1u, abort_flag, p.status)) != 0;
                    if (!ok) break;
                    tc_fence_after();
                    uint32_t r[32];
                    tc_ld_16x256b_x8(tmem_base + lane_field + (uint32_t)(kSCol0 + sb * kTile), r);
                    tc_wait_ld();
                    release_accumulator(&bars->s_empty[sb], lane);
#pragma unroll
                    for (int u = 0; u < 8; ++u)
#pragma unroll
                        for (int e = 0; e < 2; ++e) {
                            const float ta = __uint_as_float(r[4 * u + e]) * c2, tb = __uint_as_float(r[4 * u + 2 + e]) * c2;
                            if (!((mask >> (2 * u + e)) & 1u)) m_a = fmaxf(m_a, ta);
                            if (!((mask >> (16 + 2 * u + e)) & 1u)) m_b = fmaxf(m_b, tb);
                        }
                }
                if (!ok) break;
                m_a = fmaxf(m_a, __shfl_xor_sync(0xffffffffu, m_a, 1)); m_a = fmaxf(m_a, __shfl_xor_sync(0xffffffffu, m_a, 2));
                m_b = fmaxf(m_b, __shfl_xor_sync(0xffffffffu, m_b, 1)); m_b = fmaxf(m_b, __shfl_xor_sync(0xffffffffu, m_b, 2));
                const float sub_a = m_a == -INFINITY ? 0.f : m_a, sub_b = m_b == -INFINITY ? 0.f : m_b;
                // ---- pass 2: P = exp2(scale * log2(e) * S - m) as a K-major operand tile, row sums
                float l_a = 0.f, l_b = 0.f;
                win.begin(p.blocks, cur.first, cur.count, pre, lane);
                for (int j = 0; ok && j < n; ++j, ++s_no, ++p_no) {
                    const int sb = s_no & 1, pb = p_no & 1;
                    const int col = masked_op ? win.get(p.blocks, cur.first, cur.count, j, lane).col() : 0;
                    const uint32_t mask = masked_op ? block_mask(col) : 0u;
                    ok = __all_sync(0xffffffffu, mbar_wait(&bars->s_full[sb], (uint32_t)(s_no >> 1) & 1u, abort_flag, p.status)) != 0;
                    if (!ok) break;
                    tc_fence_after();
                    uint32_t r[32];
                    tc_ld_16x256b_x8(tmem_base + lane_field + (uint32_t)(kSCol0 + sb * kTile), r);
                    tc_wait_ld();
                    release_accumulator(&bars->s_empty[sb], lane);
                    uint32_t w_a[8], w_b[8];            // packed pairs: columns 8u + 2 * q4 + {0, 1}
#pragma unroll
                    for (int u = 0; u < 8; ++u) {
                        float pa[2], pb2[2];
#pragma unroll
                        for (int e = 0; e < 2; ++e) {
                            pa[e] = attn_exp2(fmaf(__uint_as_float(r[4 * u + e]), c2, -sub_a));
                            pb2[e] = attn_exp2(fmaf(__uint_as_float(r[4 * u + 2 + e]), c2, -sub_b));
                            if ((mask >> (2 * u + e)) & 1u) pa[e] = 0.f;
                            if ((mask >> (16 + 2 * u + e)) & 1u) pb2[e] = 0.f;
                            l_a += pa[e];
                            l_b += pb2[e];
                        }
                        w_a[u] = pack2<BF16>(pa[0], pa[1]);
                        w_b[u] = pack2<BF16>(pb2[0], pb2[1]);
                    }
                    // the P buffer must have been read by the MMAs of two blocks ago
                    ok = __all_sync(0xffffffffu, mbar_wait(&bars->p_empty[pb], ((uint32_t)(p_no >> 1) & 1u) ^ 1u, abort_flag, p.status)) != 0;
                    if (!ok) break;
                    uint8_t* tile = p_smem + pb * kTileBytes;
#pragma unroll
                    for (int half = 0; half < 2; ++half) {     // columns 32 * half .. 32 * half + 31
                        uint32_t ta[4] = {w_a[4 * half], w_a[4 * half + 1], w_a[4 * half + 2], w_a[4 * half + 3]};
                        uint32_t tb[4] = {w_b[4 * half], w_b[4 * half + 1], w_b[4 * half + 2], w_b[4 * half + 3]};
                        quad_transpose(ta, q4);                // now columns 32 * half + 8 * q4 .. + 7 of the row
                        quad_transpose(tb, q4);
                        const int chunk = 4 * half + q4;       // 16-byte piece of the 128-byte row
                        *reinterpret_cast<uint4*>(tile + row_a * 128 + ((chunk ^ (row_a & 7)) << 4)) = make_uint4(ta[0], ta[1], ta[2], ta[3]);
                        *reinterpret_cast<uint4*>(tile + row_b * 128 + ((chunk ^ (row_b & 7)) << 4)) = make_uint4(tb[0], tb[1], tb[2], tb[3]);
                    }
                    fence_async_shared();           // generic-proxy writes -> visible to the tensor core's reads
                    __syncwarp();
                    if (lane == 0) mbar_arrive(&bars->p_full[pb]);
                }
                if (!ok) break;
                l_a += __shfl_xor_sync(0xffffffffu, l_a, 1); l_a += __shfl_xor_sync(0xffffffffu, l_a, 2);
                l_b += __shfl_xor_sync(0xffffffffu, l_b, 1); l_b += __shfl_xor_sync(0xffffffffu, l_b, 2);
                const float inv_a = l_a > 0.f ? 1.f / l_a : 0.f, inv_b = l_b > 0.f ? 1.f / l_b : 0.f;
                // ---- end of the row: O / l
                ok = __all_sync(0xffffffffu, mbar_wait(&bars->o_full, (uint32_t)(o_no & 1), abort_flag, p.status)) != 0;
                if (!ok) break;
                tc_fence_after();
                for (int t = 0; t < p.dtiles; ++t) {
                    uint32_t r[32];
                    tc_ld_16x256b_x8(tmem_base + lane_field + (uint32_t)(t * kTile), r);
                    tc_wait_ld();
                    if (t == p.dtiles - 1) release_accumulator(&bars->o_empty, lane);
#pragma unroll
                    for (int half = 0; half < 2; ++half) {
                        uint32_t ta[4], tb[4];
#pragma unroll
                        for (int u = 0; u < 4; ++u) {
                            const int uu = 4 * half + u;
                            ta[u] = pack2<BF16>(__uint_as_float(r[4 * uu]) * inv_a, __uint_as_float(r[4 * uu + 1]) * inv_a);
                            tb[u] = pack2<BF16>(__uint_as_float(r[4 * uu + 2]) * inv_b, __uint_as_float(r[4 * uu + 3]) * inv_b);
                        }
                        quad_transpose(ta, q4);
                        quad_transpose(tb, q4);
                        const int c = t * kTile + 32 * half + 8 * q4;
                        *reinterpret_cast<uint4*>(p.o + o_row_a + c) = make_uint4(ta[0], ta[1], ta[2], ta[3]);
                        *reinterpret_cast<uint4*>(p.o + o_row_b + c) = make_uint4(tb[0], tb[1], tb[2], tb[3]);
                    }
                }
                ++o_no;
                if (q4 == 0 && p.lse) {
                    // natural-log sum of exponentials of the scaled, masked scores
                    p.lse[lse_a] = l_a > 0.f ? (m_a + log2f(l_a)) * 0.6931471805599453f : -INFINITY;
                    p.lse[lse_a + 8] = l_b > 0.f ? (m_b + log2f(l_b)) * 0.6931471805599453f : -INFINITY;
                }
            }
            pre = pre_next;
            cur.advance();
        }
    }

    // ---------------------------------------------------------------- teardown
    tc_fence_before();
    __syncthreads();
    if (warp == 1) {
        __syncwarp();
        tc_fence_after();
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"((uint32_t)kAttnTmemCols)
                     : "memory");
    }
}

}  // namespace

// Host side of bsa_attention_forward (arguments already validated by the caller).
int attention_forward(int dtype, const void* q, const void* k, const void* v, void* o, float* lse,
                      const int32_t* row_blocks, const int32_t* row_table, int64_t nnz, int64_t block_rows,
                      int64_t block_cols, int64_t batches, int64_t head_dim, float scale, int causal,
                      const uint8_t* kpm, int64_t kpm_batches, int64_t kpm_stride, uint32_t* workspace,
                      cudaStream_t stream) {
    using KernelFn = void (*)(const CUtensorMap, const CUtensorMap, const CUtensorMap, const AttnParams);
    const KernelFn kernel = dtype == BSA_DTYPE_BF16 ? attention_forward_kernel<true> : attention_forward_kernel<false>;
    AttnParams p{};
    p.dtiles = (int)(head_dim / kTile);
    p.ring = p.dtiles == 1 ? 4 : 2;
    p.ring_shift = p.dtiles == 1 ? 2 : 1;
    const int smem_bytes = 1024 + ((1 + 2 * p.ring) * p.dtiles + 2) * kTileBytes + (int)sizeof(AttnBarriers);
    // Set on every call (a per-device attribute); this and the cudaSetDevice below also bind the
    // device's primary context to the calling thread, which the driver call behind make_map needs.
    if (cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, smem_bytes) != cudaSuccess) {
        cudaGetLastError();
        return BSA_ERR_LAUNCH;
    }
    {
        int dev = 0;
        if (cudaGetDevice(&dev) != cudaSuccess || cudaSetDevice(dev) != cudaSuccess) { cudaGetLastError(); return BSA_ERR_LAUNCH; }
    }
    const int64_t seq_q = block_rows * kTile, seq_k = block_cols * kTile;
    CUtensorMap map_q, map_k, map_v;
    bool ok = make_map(&map_q, dtype, q, batches, seq_q, head_dim);
    ok &= make_map(&map_k, dtype, k, batches, seq_k, head_dim);
    ok &= make_map(&map_v, dtype, v, batches, seq_k, head_dim);
    if (!ok) return BSA_ERR_DRIVER;

    p.blocks = reinterpret_cast<const BlockDesc*>(row_blocks);
    p.table = row_table;
    p.status = workspace;
    p.nnz = (int)nnz; p.groups = (int)block_rows; p.batches = (int)batches;
    p.chunks = 1;
    p.items = (int)(batches * block_rows);
    p.seq_q = (int)seq_q; p.seq_k = (int)seq_k; p.head_dim = (int)head_dim;
    p.scale_log2 = scale * 1.4426950408889634f;
    p.causal = causal;
    p.kpm = kpm;
    p.kpm_div = kpm ? (int)(batches / kpm_batches) : 1;
    p.kpm_stride = kpm_stride;
    p.o = static_cast<uint16_t*>(o);
    p.lse = lse;
    // instruction descriptors: fp32 accumulate, fp16 / bf16 operands, M = 64; Q K^T: both operands
    // K-major, N = 64; P V: B (V tiles) with N contiguous, N = head_dim
    const uint32_t fmt = dtype == BSA_DTYPE_BF16 ? 1u : 0u;
    const uint32_t common = (1u << 4) | (fmt << 7) | (fmt << 10) | ((uint32_t)(kTile >> 4) << 24);
    p.idesc_qk = common | ((uint32_t)(kTile >> 3) << 17);
    p.idesc_pv = common | (1u << 16) | ((uint32_t)(head_dim >> 3) << 17);

    const int sms = sm_count();
    if (sms <= 0) return BSA_ERR_LAUNCH;
    const unsigned grid = (unsigned)(p.items < 2 * sms ? p.items : 2 * sms);
    p.stride_z = (int)grid / p.groups;
    p.stride_rem = (int)grid % p.groups;
    kernel<<<grid, kAttnThreads, smem_bytes, stream>>>(map_q, map_k, map_v, p);
    return launch_status();
}

bool attention_supports(int dtype, int64_t head_dim, int block) {
    return (dtype == BSA_DTYPE_F16 || dtype == BSA_DTYPE_BF16) && block == kTile && (head_dim == 64 || head_dim == 128);
}

}  // namespace bsa

extern "C" int bsa_attention_forward(int dtype, const void* q, const void* k, const void* v, void* o, float* lse,
                                     const int32_t* row_blocks, const int32_t* row_table,
                                     int64_t nnz, int64_t block_rows, int64_t block_cols, int64_t batches,
                                     int64_t head_dim, int block, float scale, int causal,
                                     const uint8_t* key_padding_mask, int64_t kpm_batches, int64_t kpm_stride,
                                     void* workspace, size_t workspace_bytes, void* stream) {
    using namespace bsa;
    if (dtype != BSA_DTYPE_F32 && dtype != BSA_DTYPE_F16 && dtype != BSA_DTYPE_BF16) return BSA_ERR_BAD_DTYPE;
    if (block != 32 && block != 64 && block != 128) return BSA_ERR_BAD_BLOCK;
    if (!q || !k || !v || !o || !row_blocks || !row_table) return BSA_ERR_NULL_POINTER;
    if (!workspace || workspace_bytes < BSA_WORKSPACE_BYTES) return BSA_ERR_WORKSPACE;
    if (nnz < 0 || block_rows <= 0 || block_cols <= 0 || batches < 0 || head_dim <= 0) return BSA_ERR_BAD_SHAPE;
    if (block_rows > 65535 || block_cols > 65535 || nnz > block_rows * block_cols) return BSA_ERR_BAD_SHAPE;
    if (!attention_supports(dtype, head_dim, block)) return dtype == BSA_DTYPE_F32 ? BSA_ERR_BAD_DTYPE : BSA_ERR_BAD_SHAPE;
    if (batches > 65535 || batches * block_rows >= ((int64_t)1 << 30) || block_rows * block >= ((int64_t)1 << 31)) return BSA_ERR_TOO_LARGE;
    if (!aligned16(q) || !aligned16(k) || !aligned16(v) || !aligned16(o)) return BSA_ERR_ALIGNMENT;
    if (key_padding_mask && (kpm_batches <= 0 || batches % kpm_batches != 0 || kpm_stride < block_cols * block))
        return BSA_ERR_BAD_SHAPE;
    if (batches == 0) return BSA_OK;
    return attention_forward(dtype, q, k, v, o, lse, row_blocks, row_table, nnz, block_rows, block_cols, batches,
                             head_dim, scale, causal, key_padding_mask, kpm_batches, kpm_stride,
                             static_cast<uint32_t*>(workspace), static_cast<cudaStream_t>(stream));
}
