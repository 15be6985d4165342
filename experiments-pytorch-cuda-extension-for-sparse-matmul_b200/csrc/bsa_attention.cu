// Fused block-sparse attention forward (sm_100a only):
//   O = softmax_rows(scale * Q K^T + masks, restricted to the layout) V
// in one kernel, so the score and probability blocks never travel through HBM.  The reference
// composes this from three launches of its matmul and softmax kernels (sdd: sparse_smm_gpu.cu:22-99,
// softmax: sparse_softmax.cu:113-155, dsd: sparse_smm_gpu.cu:101-183), each writing the
// [batch, nnz, block, block] tensor to memory; this entry point has no counterpart there and
// exists beside the three unfused operators.
//
// Work item = one block row r of one batch entry (64 query rows).  One pass over the row's
// blocks c_0 .. c_{n-1}, both products on the tensor cores (tcgen05, fp32 accumulators in TMEM):
//   S_j = Q_r K_{c_j}^T; P_j = exp(scale * S_j - m) written as a 16-bit K-major operand tile to
//   shared memory; O += P_j V_{c_j}; the row sums l accumulate next to it; at the end O / l goes
//   to global memory and lse = m + log l.
// m is a running row maximum that is raised lazily: only when a block's maximum exceeds it by more
// than 8 (in units of log2), so P never exceeds 2^8 and the rescaling of O and l by
// exp(m_old - m_new), a TMEM round trip that has to wait for the previous P V, is rare (for scores
// of similar size it happens in a row's first blocks only).  The result does not depend on when m
// is raised: O and l carry the same factor.
//
// Two kernels: head dim 64 runs as two independent pipelines per CTA (second half of this file);
// head dim 128 (one O accumulator fits into a CTA's 256 TMEM columns beside two S buffers) runs the
// kernel below.  A thread issues a tcgen05.mma, a commit or a TMA copy only every ~60-100 cycles
// whatever its size (twice that from a diverged lane: the role loops run warp-uniformly and elect a
// lane only around the instructions), so producing and issuing are spread over four warps; two
// CTAs share an SM and overlap each other's prologues and epilogues:
//   warp 0     TMA producer of Q and of every block's K tiles
//   warp 1     Q K^T issuer: S is double buffered, so Q K^T of block j + 1 runs while the softmax
//              warps work on block j; one commit per block signals both "S is ready" and "the K
//              stage is free"
//   warp 2     TMA producer of the V tiles (a K stage is free long before the block's P V: one
//              in-order producer would stretch every loop by a TMA latency)
//   warp 3     P V issuer; one commit per block signals "the P buffer and the V stage are free"
//   warps 4-7  softmax warpgroup: tcgen05.ld with the 16x256b shape (every lane owns 2 rows x 16
//              columns of a 64 x 64 block), masks, max / exp / sum, pack, stmatrix into the
//              128-byte-swizzled P tile; two register buffers, the TMEM load of block j + 1 in flight
//              while block j is worked on; at the end of a row O goes through 4x4 quad transposes
//              and 128-bit stores to global memory.
// All waits are bounded (BSA_ERR_DEVICE_TIMEOUT in the workspace word).
#include "bsa_tc_common.cuh"

namespace bsa {
namespace {

constexpr int kAttnTmemCols = 256;      // O: columns 0 .. head_dim - 1; S buffers: 128 .. 191, 192 .. 255
constexpr int kSCol0 = 128;
constexpr int kMaxRing = 4;

struct __align__(8) AttnBarriers {
    uint64_t q_full[2];
    uint64_t q_empty[2];            // the last Q K^T of the item that used the buffer has retired
    uint64_t k_full[kMaxRing];
    uint64_t qk_done[kMaxRing];     // the MMAs of one Q K^T have retired: S is ready and the K stage is free
    uint64_t v_full[kMaxRing];
    uint64_t pv_done[kMaxRing];     // the MMAs of one P V have retired: the P buffer and the V stage are free
    uint64_t s_empty[2];
    uint64_t p_full[2];
    uint64_t o_full[2], o_empty[2]; // indexed by the parity of the item
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
    int ring, ring_shift;      // K pipeline depth (a power of two) and its log2
    int vring, vring_shift;    // V pipeline depth and its log2 (there are always 2 P buffers)
    int qbufs;                 // Q buffers: 2 = the next item's Q tile set is prefetched
    float scale_log2;          // scale * log2(e)
    int causal;
    int quadrants;             // 1: the idx field of a descriptor holds a 4-bit mask of the 32 x 32 quadrants of the
                               // block that belong to the layout (bit 2 * row_half + col_half); the others are masked
    const uint8_t* kpm;        // key padding mask or nullptr
    int kpm_div;               // batch entries per mask row
    long long kpm_stride;
    uint16_t* o;
    float* lse;
    uint32_t idesc_qk, idesc_pv;
};

template <bool BF16, bool MASKED>
__global__ void __launch_bounds__(8 * 32, 2)
attention_forward_kernel(const __grid_constant__ CUtensorMap map_q, const __grid_constant__ CUtensorMap map_k,
                         const __grid_constant__ CUtensorMap map_v, const AttnParams p) {
    extern __shared__ uint8_t smem_raw[];
    uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~(uintptr_t)1023);
    // tiles: Q (qbufs x dtiles), K ring (ring x dtiles), V ring (vring x dtiles), P (2)
    const int set_bytes = p.dtiles * kTileBytes;            // one Q / K / V tile set
    uint8_t* q_smem = smem;
    uint8_t* k_smem = q_smem + p.qbufs * set_bytes;
    uint8_t* v_smem = k_smem + p.ring * set_bytes;
    uint8_t* p_smem = v_smem + p.vring * set_bytes;
    AttnBarriers* bars = reinterpret_cast<AttnBarriers*>(p_smem + 2 * kTileBytes);
    int* abort_flag = &bars->abort_flag;

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int ring_mask = p.ring - 1, vring_mask = p.vring - 1;

    if (threadIdx.x == 0) {
        for (int s = 0; s < 2; ++s) {
            mbar_init(&bars->q_full[s], 1); mbar_init(&bars->q_empty[s], 1); mbar_init(&bars->p_full[s], 4);
            mbar_init(&bars->s_empty[s], 4);
            mbar_init(&bars->o_full[s], 1); mbar_init(&bars->o_empty[s], 4);
        }
        for (int s = 0; s < kMaxRing; ++s) {
            mbar_init(&bars->k_full[s], 1); mbar_init(&bars->qk_done[s], 1);
            mbar_init(&bars->v_full[s], 1); mbar_init(&bars->pv_done[s], 1);
        }
        mbar_init(&bars->drain, 2);
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

    if (warp == 0 || warp == 2) {
        // ------------------------------------------------------------ TMA producers
        // Warp 0 loads Q and the K tiles, warp 2 the V tiles: a K stage is free again as soon as its
        // Q K^T has retired, long before the block's P V, and must not wait for it.
        const bool is_v = warp == 2;
        int kv_no = 0, q_no = 0;                   // blocks (K or V tile sets) and Q tile sets loaded so far
        bool q_prefetched = false;                 // the current item's Q tile set was requested an item ago
        bool ok = true;
        Cursor cur;
        cur.init(p, 0, true);
        BlockDesc pre = cur.valid() ? load_first_chunk(p.blocks, cur.first, cur.count, lane) : BlockDesc{0, 0};
        while (ok && cur.valid()) {
            BlockDesc pre_next{0, 0};
            if (cur.has_next()) pre_next = load_first_chunk(p.blocks, cur.next_first(), cur.next_count(), lane);
            const int n = cur.count;
            if (n > 0) {
                // Q tile set number q goes to buffer q % qbufs once the Q K^T of the item that used the
                // buffer last have retired.  With two buffers the next item's set is requested after
                // this item's K tiles (before them the request would wait for the previous item's last
                // Q K^T with nothing in flight behind it).
                auto issue_q = [&](int q, int z, int g) -> bool {        // called by the whole warp
                    const int qb = q & (p.qbufs - 1);
                    const uint32_t use = (uint32_t)(p.qbufs == 2 ? q >> 1 : q);
                    if (!__all_sync(0xffffffffu, mbar_wait(&bars->q_empty[qb], (use & 1u) ^ 1u, abort_flag, p.status))) return false;
                    if (elect_one()) {
                        mbar_expect_tx(&bars->q_full[qb], (uint32_t)set_bytes);
                        for (int t = 0; t < p.dtiles; ++t)
                            tma_load_3d(q_smem + qb * set_bytes + t * kTileBytes, &map_q, &bars->q_full[qb], t * kTile, g * kTile, z);
                    }
                    __syncwarp();
                    return true;
                };
                if (!is_v && !q_prefetched) {
                    ok = issue_q(q_no, cur.z, cur.g);
                }
                ++q_no;
                DescWindow win;
                win.begin(p.blocks, cur.first, cur.count, pre, lane);
                for (int j = 0; ok && j < n; ++j) {
                    const int col = win.get(p.blocks, cur.first, cur.count, j, lane).col();
                    // The whole warp waits for the stage and computes the copies' operands
                    // (warp-uniform code keeps them in uniform registers); an elected lane issues.
                    const int stage = is_v ? (kv_no & vring_mask) : (kv_no & ring_mask);
                    const uint32_t parity = ((uint32_t)(kv_no >> (is_v ? p.vring_shift : p.ring_shift)) & 1u) ^ 1u;
                    uint64_t* reuse = is_v ? &bars->pv_done[stage] : &bars->qk_done[stage];
                    uint64_t* full = is_v ? &bars->v_full[stage] : &bars->k_full[stage];
                    uint8_t* dst = (is_v ? v_smem : k_smem) + stage * set_bytes;
                    const CUtensorMap* map = is_v ? &map_v : &map_k;
                    ok = __all_sync(0xffffffffu, mbar_wait(reuse, parity, abort_flag, p.status)) != 0;
                    if (ok && elect_one()) {
                        mbar_expect_tx(full, (uint32_t)set_bytes);
                        for (int t = 0; t < p.dtiles; ++t)
                            tma_load_3d(dst + t * kTileBytes, map, full, t * kTile, col * kTile, cur.z);
                    }
                    __syncwarp();
                    ++kv_no;
                }
                q_prefetched = false;
                if (ok && !is_v && p.qbufs == 2 && cur.has_next() && cur.next_count() > 0) {
                    ok = issue_q(q_no, cur.next_z(), cur.next_group());        // q_no already counts this item
                    q_prefetched = true;
                }
            }
            pre = pre_next;
            cur.advance();
        }
        if (lane == 0 && *(volatile int*)abort_flag) {
            let_copies_land();      // (issued by this warp; see the helper)
        }
        __syncwarp();
    } else if (warp == 1) {
        // ------------------------------------------------------------ Q K^T issuer
        // The S tiles (blocks) of a CTA are numbered in the order they are produced; tile s goes to
        // S buffer s & 1, so Q K^T of block j + 1 runs while the softmax warps work on block j.
        {
            int s_no = 0, q_no = 0;
            bool ok = true;
            const uint32_t idesc_qk = p.idesc_qk;
            Cursor cur;
            cur.init(p, 0, true);
            for (; ok && cur.valid(); cur.advance()) {
                const int n = cur.count;
                if (n == 0) continue;               // empty row: the softmax warps write zeros on their own
                const int qb = q_no & (p.qbufs - 1);
                ok = __all_sync(0xffffffffu, mbar_wait(&bars->q_full[qb], (uint32_t)(p.qbufs == 2 ? q_no >> 1 : q_no) & 1u, abort_flag, p.status)) != 0;
                if (!ok) break;
                const int s_end = s_no + n;
                for (int s = s_no; s < s_end; ++s) {
                    const int ks = s & ring_mask, sb = s & 1;
                    ok = __all_sync(0xffffffffu, mbar_wait(&bars->k_full[ks], (uint32_t)(s >> p.ring_shift) & 1u, abort_flag, p.status)) != 0;
                    if (ok) ok = __all_sync(0xffffffffu, mbar_wait(&bars->s_empty[sb], ((uint32_t)(s >> 1) & 1u) ^ 1u, abort_flag, p.status)) != 0;
                    if (!ok) break;
                    tc_fence_after();
                    const uint32_t d = tmem_base + (uint32_t)(kSCol0 + sb * kTile);
                    if (elect_one()) {
                        for (int t = 0; t < p.dtiles; ++t) {
                            const uint64_t da = make_tile_desc(smem_u32(q_smem + qb * set_bytes + t * kTileBytes), false);
                            const uint64_t db = make_tile_desc(smem_u32(k_smem + ks * set_bytes + t * kTileBytes), false);
#pragma unroll
                            for (int kk = 0; kk < kTile / 16; ++kk)
                                tc_mma_f16(d, da + (uint64_t)(kk * 2), db + (uint64_t)(kk * 2), idesc_qk, (t > 0 || kk > 0) ? 1u : 0u);
                        }
                        tc_commit(&bars->qk_done[ks]);
                    }
                    __syncwarp();
                }
                if (!ok) break;
                if (elect_one()) tc_commit(&bars->q_empty[qb]);      // the last read of this Q buffer has been issued
                __syncwarp();
                s_no = s_end;
                ++q_no;
            }
            // All MMAs issued by the elected lane (the same one every time: the election is
            // deterministic for a converged warp) must have retired before TMEM is freed.
            if (elect_one()) {
                tc_commit(&bars->drain);
                mbar_wait(&bars->drain, 0, abort_flag, p.status);
            }
        }
        __syncwarp();
    } else if (warp == 3) {
        // ------------------------------------------------------------ P V issuer
        {
            int p_no = 0, o_no = 0;
            bool ok = true;
            const uint32_t idesc_pv = p.idesc_pv;
            Cursor cur;
            cur.init(p, 0, true);
            for (; ok && cur.valid(); cur.advance()) {
                const int n = cur.count;
                if (n == 0) continue;
                for (int j = 0; ok && j < n; ++j, ++p_no) {
                    const int pb = p_no & 1, vs = p_no & vring_mask;
                    // the accumulators are free once the item before has been read out (its barrier: its parity)
                    if (j == 0 && o_no > 0)
                        ok = __all_sync(0xffffffffu, mbar_wait(&bars->o_empty[(o_no - 1) & 1], (uint32_t)((o_no - 1) >> 1) & 1u, abort_flag, p.status)) != 0;
                    if (ok) ok = __all_sync(0xffffffffu, mbar_wait(&bars->v_full[vs], (uint32_t)(p_no >> p.vring_shift) & 1u, abort_flag, p.status)) != 0;
                    if (ok) ok = __all_sync(0xffffffffu, mbar_wait(&bars->p_full[pb], (uint32_t)(p_no >> 1) & 1u, abort_flag, p.status)) != 0;
                    if (!ok) break;
                    tc_fence_after();
                    // O += P_j V_{c_j}: A = P (K-major), B = V tiles (N contiguous), N = head_dim
                    const uint64_t da = make_tile_desc(smem_u32(p_smem + pb * kTileBytes), false);
                    const uint64_t db = make_tile_desc(smem_u32(v_smem + vs * set_bytes), true);
                    const uint32_t d = tmem_base;
                    if (elect_one()) {
#pragma unroll
                        for (int kk = 0; kk < kTile / 16; ++kk)
                            tc_mma_f16(d, da + (uint64_t)(kk * 2), db + (uint64_t)(kk * (2048 >> 4)), idesc_pv,
                                       (j > 0 || kk > 0) ? 1u : 0u);
                        tc_commit(&bars->pv_done[vs]);
                        if (j == n - 1) tc_commit(&bars->o_full[o_no & 1]);
                    }
                    __syncwarp();
                }
                ++o_no;
            }
            if (elect_one()) {
                tc_commit(&bars->drain);
                mbar_wait(&bars->drain, 0, abort_flag, p.status);
            }
        }
        __syncwarp();
    } else {
        // ------------------------------------------------------------ softmax warps
        const int quad = warp & 3;                  // TMEM sub-partition this warp may read
        const int q4 = lane & 3;                    // position in the quad: columns 8u + 2 * q4 + {0, 1}
        const int row_a = quad * 16 + (lane >> 2);  // this lane's two rows of the 64-row block
        const uint32_t lane_field = (uint32_t)(quad * 32) << 16;
        // MASKED = false: no causal or key-padding mask, all mask tests fold away
        const bool masked_op = MASKED && (p.causal != 0 || p.kpm != nullptr || p.quadrants != 0);
        int s_no = 0, o_no = 0;                     // S tiles and non-empty items before the current item
        bool ok = true;
        Cursor cur;
        cur.init(p, 0, true);
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
                {
                    for (int c = q4 * 8; c < p.head_dim; c += 32) {
                        *reinterpret_cast<uint4*>(p.o + o_row_a + c) = make_uint4(0u, 0u, 0u, 0u);
                        *reinterpret_cast<uint4*>(p.o + o_row_b + c) = make_uint4(0u, 0u, 0u, 0u);
                    }
                    if (q4 == 0 && p.lse) { p.lse[lse_a] = -INFINITY; p.lse[lse_a + 8] = -INFINITY; }
                }
            } else {
                const uint8_t* kpm_row = p.kpm ? p.kpm + (size_t)(cur.z / p.kpm_div) * p.kpm_stride : nullptr;
                const int qpos_a = cur.g * kTile + row_a;
                // Bits 0-15: columns (u, e) of row a that are masked in block `col`; bits 16-31: row b.
                auto block_mask = [&](const BlockDesc& desc) -> uint32_t {
                    const int col = desc.col();
                    uint32_t m = 0;
                    if (p.quadrants) {
                        // this lane's rows lie in row half quad / 2; its columns 8u + .. in column half u / 4
                        const uint32_t present = (uint32_t)desc.idx >> (2 * (quad >> 1));
                        if (!(present & 1u)) m |= 0x00FF00FFu;
                        if (!(present & 2u)) m |= 0xFF00FF00u;
                    }
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
                const bool flip = c2 < 0.f;
                // ---- one pass over the row's blocks with a running row maximum m (in units of
                // log2: t = scale * log2(e) * s).  P_j = exp2(t_j - m) goes to shared memory as a
                // K-major operand tile, O += P_j V_j accumulates in TMEM, l sums the P's.  m is only
                // raised when a block's maximum exceeds it by more than kSlack (P stays <= 2^kSlack,
                // exact in fp32 sums and well inside the 16-bit range); raising it rescales O in TMEM
                // and l by exp2(m_old - m_new), which needs this group's previous P V to have retired.
                constexpr float kSlack = 8.f;
                float m_a = -INFINITY, m_b = -INFINITY;
                // row sums: per row two independent two-wide accumulators (even / odd column units), added up at the end
                uint64_t la2[2] = {0ull, 0ull}, lb2[2] = {0ull, 0ull};
                DescWindow win;
                win.begin(p.blocks, cur.first, cur.count, pre, lane);
                // P leaves through stmatrix: the 16x256b TMEM load hands out the m8n8 fragment layout, so the packed
                // words of column units 2k, 2k + 1 of the lane's two rows are the four matrices of one instruction.
                // Lane -> row address of its matrix: matrix i = lane / 8 holds rows (i & 1) * 8 .. of unit 2k + (i >> 1).
                // Its address in unit 2k is row * 128 + (((2k + (i >> 1)) ^ (row & 7)) << 4) = p_off ^ (k << 5): bits 5-6
                // carry 2k ^ (row & 6), bit 4 the unit's parity, and the tiles are 1024-byte aligned.
                const int sm_row = quad * 16 + ((lane >> 3) & 1) * 8 + (lane & 7);
                const uint32_t p_off = (uint32_t)(sm_row * 128) + ((((uint32_t)(lane >> 4)) ^ (uint32_t)(sm_row & 7)) << 4);
                const float c2abs = fabsf(c2);
                auto load = [&](uint32_t (&r)[32], int t) -> bool {       // wait for S tile t, start loading it
                    const int s = s_no + t;
                    if (!__all_sync(0xffffffffu, mbar_wait(&bars->qk_done[s & ring_mask], (uint32_t)(s >> p.ring_shift) & 1u,
                                                           abort_flag, p.status)))
                        return false;
                    tc_fence_after();
                    tc_ld_16x256b_x8(tmem_base + lane_field + (uint32_t)(kSCol0 + (s & 1) * kTile), r);
                    return true;
                };
                auto loaded = [&](int t) {                                 // tile t is in registers: free its buffer
                    tc_wait_ld();
                    release_accumulator(&bars->s_empty[(s_no + t) & 1], lane);
                };
                // Masked elements (above the diagonal, padded keys, quadrants outside a block-32 layout) are
                // overwritten in registers by -inf (+inf for a negative scale) before the common code runs:
                // they then lose every maximum and their exp2 is exactly 0 (the host keeps the scale factor
                // away from 0, so inf * scale is never NaN).  One copy of the softmax code for both kernel
                // variants: separate masked code cost the softmax warps, which bound the kernel, 40 % more
                // instructions, and two copies cost registers.
                // (the mask of a block is computed before the wait for its S tile: off the critical chain)
                auto mask_of = [&](int t) -> uint32_t {
                    if (MASKED && masked_op) return block_mask(win.get(p.blocks, cur.first, cur.count, t, lane));
                    return 0u;
                };
                auto process = [&](uint32_t (&r)[32], int t, const uint32_t mask) -> bool {
                    if (MASKED && masked_op) {
                        if (mask != 0u) {
                            const uint32_t gone = flip ? 0x7F800000u : 0xFF800000u;
#pragma unroll
                            for (int i = 0; i < 16; ++i) {
                                const int u = i >> 1, e = i & 1;
                                if ((mask >> i) & 1u) r[4 * u + e] = gone;
                                if ((mask >> (16 + i)) & 1u) r[4 * u + 2 + e] = gone;
                            }
                        }
                    }
                    const int s = s_no + t;                                  // tile number = P buffer number
                    // block maxima of the raw scores (for a negative scale: of their negatives)
                    float x_a, x_b;
                    {
                        // two chains per row (even / odd column units) of three-input maxima
                        float a0 = -INFINITY, a1 = -INFINITY, b0 = -INFINITY, b1 = -INFINITY;
                        if (!flip) {
#pragma unroll
                            for (int u = 0; u < 8; u += 2) {
                                a0 = fmax3(a0, __uint_as_float(r[4 * u]), __uint_as_float(r[4 * u + 1]));
                                b0 = fmax3(b0, __uint_as_float(r[4 * u + 2]), __uint_as_float(r[4 * u + 3]));
                                a1 = fmax3(a1, __uint_as_float(r[4 * u + 4]), __uint_as_float(r[4 * u + 5]));
                                b1 = fmax3(b1, __uint_as_float(r[4 * u + 6]), __uint_as_float(r[4 * u + 7]));
                            }
                            x_a = fmaxf(a0, a1); x_b = fmaxf(b0, b1);
                        } else {
                            a0 = a1 = b0 = b1 = INFINITY;
#pragma unroll
                            for (int u = 0; u < 8; u += 2) {
                                a0 = fmin3(a0, __uint_as_float(r[4 * u]), __uint_as_float(r[4 * u + 1]));
                                b0 = fmin3(b0, __uint_as_float(r[4 * u + 2]), __uint_as_float(r[4 * u + 3]));
                                a1 = fmin3(a1, __uint_as_float(r[4 * u + 4]), __uint_as_float(r[4 * u + 5]));
                                b1 = fmin3(b1, __uint_as_float(r[4 * u + 6]), __uint_as_float(r[4 * u + 7]));
                            }
                            x_a = -fminf(a0, a1); x_b = -fminf(b0, b1);
                        }
                    }
                    x_a = fmaxf(x_a, __shfl_xor_sync(0xffffffffu, x_a, 1)); x_a = fmaxf(x_a, __shfl_xor_sync(0xffffffffu, x_a, 2));
                    x_b = fmaxf(x_b, __shfl_xor_sync(0xffffffffu, x_b, 1)); x_b = fmaxf(x_b, __shfl_xor_sync(0xffffffffu, x_b, 2));
                    x_a = x_a == -INFINITY ? -INFINITY : x_a * c2abs;       // maxima of t over the block
                    x_b = x_b == -INFINITY ? -INFINITY : x_b * c2abs;
                    const int pb = s & 1;
                    if (t == 0) {
                        m_a = x_a; m_b = x_b;                                 // the row's first P V overwrites O
                    } else {
                        // raise a row's maximum only when it is overdue (or was -inf: nothing kept yet)
                        const bool up_a = x_a > m_a + kSlack || (m_a == -INFINITY && x_a > -INFINITY);
                        const bool up_b = x_b > m_b + kSlack || (m_b == -INFINITY && x_b > -INFINITY);
                        if (__any_sync(0xffffffffu, up_a || up_b)) {
                            const float al_a = !up_a ? 1.f : (m_a == -INFINITY ? 0.f : attn_exp2(m_a - x_a));
                            const float al_b = !up_b ? 1.f : (m_b == -INFINITY ? 0.f : attn_exp2(m_b - x_b));
                            if (up_a) { m_a = x_a; const uint64_t f = f2_pack(al_a, al_a); la2[0] = f2_mul(la2[0], f); la2[1] = f2_mul(la2[1], f); }
                            if (up_b) { m_b = x_b; const uint64_t f = f2_pack(al_b, al_b); lb2[0] = f2_mul(lb2[0], f); lb2[1] = f2_mul(lb2[1], f); }
                            // O is complete up to the previous tile once that tile's P V has retired
                            const int prev = s - 1;
                            if (!__all_sync(0xffffffffu, mbar_wait(&bars->pv_done[prev & vring_mask],
                                                                   (uint32_t)(prev >> p.vring_shift) & 1u, abort_flag, p.status)))
                                return false;
                            tc_fence_after();
                            for (int c = 0; c < p.head_dim; c += 16) {
                                uint32_t o[8];
                                tc_ld_16x256b_x2(tmem_base + lane_field + (uint32_t)c, o);
                                tc_wait_ld();
#pragma unroll
                                for (int u = 0; u < 2; ++u) {
                                    o[4 * u] = __float_as_uint(__uint_as_float(o[4 * u]) * al_a);
                                    o[4 * u + 1] = __float_as_uint(__uint_as_float(o[4 * u + 1]) * al_a);
                                    o[4 * u + 2] = __float_as_uint(__uint_as_float(o[4 * u + 2]) * al_b);
                                    o[4 * u + 3] = __float_as_uint(__uint_as_float(o[4 * u + 3]) * al_b);
                                }
                                tc_st_16x256b_x2(tmem_base + lane_field + (uint32_t)c, o);
                            }
                            tc_wait_st();
                            tc_fence_before();      // ordered before the P V this block's arrival releases
                        }
                    }
                    const float sub_a = m_a == -INFINITY ? 0.f : m_a, sub_b = m_b == -INFINITY ? 0.f : m_b;
                    // the P buffer must have been read by the MMAs that used it last (those of tile s - 2)
                    if (s >= 2 && !__all_sync(0xffffffffu, mbar_wait(&bars->pv_done[(s - 2) & vring_mask],
                                                                     (uint32_t)((s - 2) >> p.vring_shift) & 1u, abort_flag, p.status)))
                        return false;
                    // P = exp2(c2 * s - m): per pair of columns one two-wide FMA, two exp2, one two-wide add into the
                    // row sum and one pack; four stmatrix write the lane's 32 values into the swizzled tile
                    const uint32_t tile = smem_u32(p_smem + pb * kTileBytes) + p_off;
                    const uint64_t c2p = f2_pack(c2, c2), na = f2_pack(-sub_a, -sub_a), nb = f2_pack(-sub_b, -sub_b);
#pragma unroll
                    for (int k = 0; k < 4; ++k) {
                        uint32_t w[4];              // matrices (unit 2k, row a), (2k, row b), (2k + 1, a), (2k + 1, b)
#pragma unroll
                        for (int i = 0; i < 4; ++i) {
                            const int u = 2 * k + (i >> 1), h = i & 1;
                            const uint64_t t2 = f2_fma(f2_pack(__uint_as_float(r[4 * u + 2 * h]), __uint_as_float(r[4 * u + 2 * h + 1])),
                                                       c2p, h ? nb : na);
                            float e0, e1;
                            f2_unpack(t2, e0, e1);
                            e0 = attn_exp2(e0); e1 = attn_exp2(e1);
                            if (h) lb2[i >> 1] = f2_add(lb2[i >> 1], f2_pack(e0, e1));
                            else   la2[i >> 1] = f2_add(la2[i >> 1], f2_pack(e0, e1));
                            w[i] = pack2<BF16>(e0, e1);
                        }
                        stmatrix_x4(tile ^ (uint32_t)(k << 5), w[0], w[1], w[2], w[3]);
                    }
                    fence_async_shared();           // generic-proxy writes -> visible to the tensor core's reads
                    __syncwarp();
                    if (lane == 0) mbar_arrive(&bars->p_full[pb]);
                    return true;
                };
                {
                    // The TMEM load of block j + 1 is in flight while block j is worked on (two
                    // register buffers, loop unrolled by two).
                    uint32_t ra[32], rb[32];
                    uint32_t ma = mask_of(0), mb = 0u;
                    ok = load(ra, 0);
                    for (int t = 0; ok && t < n; t += 2) {
                        loaded(t);
                        if (t + 1 < n) { mb = mask_of(t + 1); ok = load(rb, t + 1); }
                        if (!process(ra, t, ma)) ok = false;
                        if (!ok || t + 1 >= n) break;
                        loaded(t + 1);
                        if (t + 2 < n) { ma = mask_of(t + 2); ok = load(ra, t + 2); }
                        if (!process(rb, t + 1, mb)) ok = false;
                    }
                }
                s_no += n;
                if (!ok) break;
                float l_a, l_b;
                {
                    float x0, x1, y0, y1;
                    f2_unpack(f2_add(la2[0], la2[1]), x0, x1);
                    f2_unpack(f2_add(lb2[0], lb2[1]), y0, y1);
                    l_a = x0 + x1; l_b = y0 + y1;
                }
                l_a += __shfl_xor_sync(0xffffffffu, l_a, 1); l_a += __shfl_xor_sync(0xffffffffu, l_a, 2);
                l_b += __shfl_xor_sync(0xffffffffu, l_b, 1); l_b += __shfl_xor_sync(0xffffffffu, l_b, 2);
                {
                    // ---- end of the row: O / l
                    const float inv_a = l_a > 0.f ? __frcp_rn(l_a) : 0.f, inv_b = l_b > 0.f ? __frcp_rn(l_b) : 0.f;
                    ok = __all_sync(0xffffffffu, mbar_wait(&bars->o_full[o_no & 1], (uint32_t)(o_no >> 1) & 1u, abort_flag, p.status)) != 0;
                    if (!ok) break;
                    tc_fence_after();
                    for (int c = 0; c < p.head_dim; c += 32) {
                        uint32_t r0[16];
                        tc_ld_16x256b_x4(tmem_base + lane_field + (uint32_t)c, r0);
                        tc_wait_ld();
                        if (c + 32 >= p.head_dim) release_accumulator(&bars->o_empty[o_no & 1], lane);
                        uint32_t ta[4], tb[4];
#pragma unroll
                        for (int u = 0; u < 4; ++u) {
                            // a row without an unmasked score gets zeros whatever its accumulator holds
                            ta[u] = pack2<BF16>(inv_a > 0.f ? __uint_as_float(r0[4 * u]) * inv_a : 0.f,
                                                inv_a > 0.f ? __uint_as_float(r0[4 * u + 1]) * inv_a : 0.f);
                            tb[u] = pack2<BF16>(inv_b > 0.f ? __uint_as_float(r0[4 * u + 2]) * inv_b : 0.f,
                                                inv_b > 0.f ? __uint_as_float(r0[4 * u + 3]) * inv_b : 0.f);
                        }
                        quad_transpose(ta, q4);         // now columns c + 8 * q4 .. + 7 of the row
                        quad_transpose(tb, q4);
                        *reinterpret_cast<uint4*>(p.o + o_row_a + c + 8 * q4) = make_uint4(ta[0], ta[1], ta[2], ta[3]);
                        *reinterpret_cast<uint4*>(p.o + o_row_b + c + 8 * q4) = make_uint4(tb[0], tb[1], tb[2], tb[3]);
                    }
                    if (q4 == 0 && p.lse) {
                        // natural-log sum of exponentials of the scaled, masked scores
                        p.lse[lse_a] = l_a > 0.f ? (m_a + __log2f(l_a)) * 0.6931471805599453f : -INFINITY;
                        p.lse[lse_a + 8] = l_b > 0.f ? (m_b + __log2f(l_b)) * 0.6931471805599453f : -INFINITY;
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
    if (warp == 1) {
        __syncwarp();
        tc_fence_after();
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"((uint32_t)kAttnTmemCols)
                     : "memory");
    }
}

// ---------------------------------------------------------------------------------------------
// Head dim 64: two independent pipelines per CTA.
//
// A pipeline is a producer warp, an issuer warp and a softmax warpgroup with their own shared-memory
// tiles (Q, three K stages, two V stages), their own S and P buffers and O accumulator in tensor
// memory and their own barriers; it walks its own block rows (pipeline number = 2 * CTA + g of
// 2 * grid pipelines).  Nothing is shared between the two pipelines of a CTA but the TMEM
// allocation, and two CTAs share an SM: four block rows are in flight per SM, each at its own
// point of its row, so the end of one row (normalising and writing O) overlaps the others' tiles.
// (An earlier version let two softmax groups share a row, with alternate tiles: the hand-overs
// between the groups, the in-order producers and issuers and the merge of the two partial results
// at the end of a row serialised the CTA; with every MMA, exponential and copy removed it still
// took 60 % of its time.)
//
// Tensor memory.  An M = 64 accumulator occupies lanes 0-15 of each 32-lane quarter; a second one
// fits into lanes 16-31 of the same columns (lane offset 16 in the MMA's D address and in the
// 16-lane tcgen05.ld / st shapes).  The 128 columns of a pipeline hold
//   columns   0 ..  63   lanes 0-15: O            lanes 16-31: S buffer 0
//   columns  64 .. 127   lanes 0-15: P buffers 0, 1 (32 columns each, 16-bit)   lanes 16-31: S buffer 1
// so S is double buffered (Q K^T runs two tiles ahead of the softmax warps) and P never touches
// shared memory: the softmax warps write it with one tcgen05.st per tile and P V takes its A
// operand from tensor memory.  (A TMEM A operand is only used at lane offset 0 together with a D
// at lane offset 0; a D at offset 16 with a TMEM A raised "misaligned address" in a probe.)
//
// A hand-over through an mbarrier costs about 200 cycles (arrive -> the waiter runs again), a test
// of a barrier that is already complete 100-250, a tcgen05.ld about 300; a tile's arithmetic takes
// 800.  So per tile the softmax warps test the barriers they are going to need ahead of time
// (non-blocking test, result consumed later), and request the next tile's S from tensor memory
// before they write this tile's P.
//   warps 0, 2   producer of pipeline 0, 1: Q of the row, then K(u), V(u - 3), ...
//   warps 1, 3   issuer: Q K^T of tile u (S buffer u & 1), then P V of tile u - 2
//   warps 4-7, 8-11   softmax warpgroup: S -> registers, masks, lazily raised running maximum,
//                P = exp2(..) packed into tensor memory, row sums; at the end of the row O / l and
//                the log-sum-exp go to global memory.
constexpr int kPipeTiles = 6;                   // Q, K x 3, V x 2
constexpr int kPipeKRing = 3;
constexpr int kPipeDescs = 8;
constexpr int kPipeRows = 8;
struct __align__(16) PipeBarriers {
    uint64_t q_full[2], q_empty[2];             // [pipeline]
    uint64_t k_full[2][kPipeKRing], qk_done[2][kPipeKRing];   // [pipeline][K stage]: qk_done = S is ready and the K stage is free
    uint64_t v_full[2][2], pv_done[2][2];       // [pipeline][tile & 1]: pv_done = the P buffer and the V stage are free
    uint64_t s_empty[2][2], p_full[2][2];       // [pipeline][tile & 1]
    uint64_t o_full[2], o_empty[2];
    uint64_t drain;
    uint32_t tmem_base;
    int abort_flag;
    BlockDesc descs[2][kPipeDescs];             // [pipeline][tile & 7]: written by the producer for the softmax warps
    uint64_t row_full[2][kPipeRows];            // [pipeline][row & 7]: the row's entry in `rows` is valid
    int4 rows[2][kPipeRows];                    // (batch entry, block row, blocks, -): written by the producer; blocks = 0: no more rows
};

// Position of a tile in the ring of three K stages (every role counts the tiles it has handled).
struct KRing {
    int stage = 0;
    uint32_t use = 0;                           // parity of the number of times the ring has wrapped
    __device__ __forceinline__ void next() { if (++stage == kPipeKRing) { stage = 0; use ^= 1u; } }
};

template <bool BF16, bool MASKED>
__global__ void __launch_bounds__(12 * 32, 2)
attention_forward_pipes_kernel(const __grid_constant__ CUtensorMap map_q, const __grid_constant__ CUtensorMap map_k,
                               const __grid_constant__ CUtensorMap map_v, const AttnParams p) {
    extern __shared__ uint8_t smem_raw[];
    uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~(uintptr_t)1023);
    PipeBarriers* bars = reinterpret_cast<PipeBarriers*>(smem + 2 * kPipeTiles * kTileBytes);
    int* abort_flag = &bars->abort_flag;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int g = warp < 4 ? warp >> 1 : (warp - 4) >> 2;          // pipeline of this warp
    uint8_t* q_smem = smem + g * kPipeTiles * kTileBytes;
    uint8_t* k_smem = q_smem + kTileBytes;
    uint8_t* v_smem = k_smem + kPipeKRing * kTileBytes;

    if (threadIdx.x == 0) {
        for (int i = 0; i < 2; ++i) {
            mbar_init(&bars->q_full[i], 1); mbar_init(&bars->q_empty[i], 1);
            for (int s = 0; s < kPipeKRing; ++s) { mbar_init(&bars->k_full[i][s], 1); mbar_init(&bars->qk_done[i][s], 1); }
            for (int s = 0; s < 2; ++s) {
                mbar_init(&bars->v_full[i][s], 1); mbar_init(&bars->pv_done[i][s], 1);
                mbar_init(&bars->s_empty[i][s], 4); mbar_init(&bars->p_full[i][s], 4);
            }
            mbar_init(&bars->o_full[i], 1); mbar_init(&bars->o_empty[i], 4);
            for (int s = 0; s < kPipeRows; ++s) mbar_init(&bars->row_full[i][s], 1);
        }
        mbar_init(&bars->drain, 2);
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
    const uint32_t o_tmem = tmem_base + (uint32_t)(g * 128);               // O: lanes 0-15 of columns 0 .. 63
    const uint32_t s_tmem = o_tmem + (16u << 16);                          // S buffer b: lanes 16-31 of columns 64 b ..
    const uint32_t p_tmem = o_tmem + 64u;                                  // P buffer b: lanes 0-15 of columns 64 + 32 b ..
    const int walker = 2 * (int)blockIdx.x + g, walkers = 2 * (int)gridDim.x;

    if (warp == 0 || warp == 2) {
        // ------------------------------------------------------------ producer
        // Order within a row: K(u), V(u - 3), the order in which their stages become free (Q K^T runs two
        // tiles ahead of the softmax warps, P V one tile behind them); the V tiles of the row's last three
        // blocks follow its last K tile, as the issuer finishes a row's P V before it starts on the next
        // row.  The stages are numbered through the rows, so Q and the first K tiles of the next row are on
        // their way while the softmax warps work on the last tiles of this one.
        int t0 = 0, i_no = 0;                       // tiles and non-empty rows before the current row
        KRing kr;                                   // stage of the next K tile
        int vq_col[3] = {0, 0, 0};                  // key blocks of tiles u - 3, u - 2, u - 1
        bool ok = true;
        Cursor cur;
        cur.init_as(p, walker, walkers, 0, true);
        BlockDesc pre = cur.valid() ? load_first_chunk(p.blocks, cur.first, cur.count, lane) : BlockDesc{0, 0};
        auto load_v = [&](int t, int col, int z) -> bool {
            const int st = t & 1;
            if (!__all_sync(0xffffffffu, mbar_wait(&bars->pv_done[g][st], ((uint32_t)(t >> 1) & 1u) ^ 1u, abort_flag, p.status))) return false;
            if (elect_one()) {
                mbar_expect_tx(&bars->v_full[g][st], (uint32_t)kTileBytes);
                tma_load_3d(v_smem + st * kTileBytes, &map_v, &bars->v_full[g][st], 0, col * kTile, z);
            }
            __syncwarp();
            return true;
        };
        while (ok && cur.valid()) {
            BlockDesc pre_next{0, 0};
            if (cur.has_next()) pre_next = load_first_chunk(p.blocks, cur.next_first(), cur.next_count(), lane);
            const int n = cur.count;
            if (n == 0) {
                // a block row without blocks: zeros, lse = -inf (the other roles never see the row)
                const size_t row0 = (size_t)cur.z * p.seq_q + (size_t)cur.g * kTile;
                for (int c = lane; c < kTile * kTile / 8; c += 32)
                    reinterpret_cast<uint4*>(p.o + row0 * kTile)[c] = make_uint4(0u, 0u, 0u, 0u);
                if (p.lse) { p.lse[row0 + lane] = -INFINITY; p.lse[row0 + 32 + lane] = -INFINITY; }
            } else {
                // Q once the last Q K^T of the row before has retired
                ok = __all_sync(0xffffffffu, mbar_wait(&bars->q_empty[g], ((uint32_t)i_no & 1u) ^ 1u, abort_flag, p.status)) != 0;
                if (ok && elect_one()) {
                    // The row's entry for the issuer and the softmax warps: they are at most three rows behind
                    // (the wait above: the softmax warps have taken the S tile two tiles before that row's last).
                    bars->rows[g][i_no & (kPipeRows - 1)] = make_int4(cur.z, cur.g, n, 0);
                    mbar_arrive(&bars->row_full[g][i_no & (kPipeRows - 1)]);
                    mbar_expect_tx(&bars->q_full[g], (uint32_t)kTileBytes);
                    tma_load_3d(q_smem, &map_q, &bars->q_full[g], 0, cur.g * kTile, cur.z);
                }
                __syncwarp();
                DescWindow win;
                win.begin(p.blocks, cur.first, cur.count, pre, lane);
                for (int j = 0; ok && j < n; ++j) {
                    const BlockDesc desc = win.get(p.blocks, cur.first, cur.count, j, lane);
                    const int col = desc.col();
                    const int u = t0 + j;
                    ok = __all_sync(0xffffffffu, mbar_wait(&bars->qk_done[g][kr.stage], kr.use ^ 1u, abort_flag, p.status)) != 0;
                    if (ok && elect_one()) {
                        // The softmax warps take the tile's descriptor (key block, quadrant bits) from here: they
                        // read it once S of the tile is ready and before they hand the S buffer back, the K stage
                        // is refilled three tiles on, Q K^T runs two tiles ahead of them: slot u & 7 is free.
                        bars->descs[g][u & (kPipeDescs - 1)] = desc;
                        mbar_expect_tx(&bars->k_full[g][kr.stage], (uint32_t)kTileBytes);
                        tma_load_3d(k_smem + kr.stage * kTileBytes, &map_k, &bars->k_full[g][kr.stage], 0, col * kTile, cur.z);
                    }
                    __syncwarp();
                    kr.next();
                    if (ok && j >= 3) ok = load_v(u - 3, vq_col[0], cur.z);
                    vq_col[0] = vq_col[1]; vq_col[1] = vq_col[2]; vq_col[2] = col;
                }
                for (int r = n < 3 ? 3 - n : 0; ok && r < 3; ++r) ok = load_v(t0 + n - 3 + r, vq_col[r], cur.z);
                t0 += n;
                ++i_no;
            }
            pre = pre_next;
            cur.advance();
        }
        if (ok && elect_one()) {                    // no more rows
            bars->rows[g][i_no & (kPipeRows - 1)] = make_int4(0, 0, 0, 0);
            mbar_arrive(&bars->row_full[g][i_no & (kPipeRows - 1)]);
        }
        __syncwarp();
        if (lane == 0 && *(volatile int*)abort_flag) {
            let_copies_land();      // (issued by this warp; see the helper)
        }
        __syncwarp();
    } else if (warp == 1 || warp == 3) {
        // ------------------------------------------------------------ issuer
        // Order within a row: Q K^T of tile u, then P V of tile u - 2; the row's last two P V follow its last
        // Q K^T, before the next row's first Q K^T (which would otherwise keep the end of this row -- the
        // softmax warps wait for the last P V to read O out -- behind the arrival of the next row's Q).  The
        // events it waits for come in this order: S(u - 2) is in the softmax warps' registers when they start
        // on tile u - 2 (S buffer u & 1 is free), their P(u - 2) is complete when they are done with it.
        const uint32_t idesc_qk = p.idesc_qk, idesc_pv = p.idesc_pv;
        const uint64_t q_desc = make_tile_desc(smem_u32(q_smem), false);
        const uint64_t k_desc = make_tile_desc(smem_u32(k_smem), false);
        const uint64_t v_desc = make_tile_desc(smem_u32(v_smem), true);
        int t0 = 0, i_no = 0;                       // tiles and non-empty rows before the current row
        KRing kr;
        bool ok = true;
        auto issue_pv = [&](int t, int row, bool first, bool last) -> bool {       // O (+)= P V of tile t
            const int b = t & 1;
            // the accumulator is free once the row before has been read out
            if (first && row > 0 &&
                !__all_sync(0xffffffffu, mbar_wait(&bars->o_empty[g], (uint32_t)(row - 1) & 1u, abort_flag, p.status)))
                return false;
            if (!__all_sync(0xffffffffu, mbar_wait(&bars->v_full[g][b], (uint32_t)(t >> 1) & 1u, abort_flag, p.status))) return false;
            if (!__all_sync(0xffffffffu, mbar_wait(&bars->p_full[g][b], (uint32_t)(t >> 1) & 1u, abort_flag, p.status))) return false;
            tc_fence_after();
            const uint64_t db = v_desc + (uint64_t)((b * kTileBytes) >> 4);
            const uint32_t a = p_tmem + (uint32_t)(32 * b);
            if (elect_one()) {
#pragma unroll
                for (int kk = 0; kk < kTile / 16; ++kk)
                    tc_mma_f16_ts(o_tmem, a + (uint32_t)(8 * kk), db + (uint64_t)(kk * (2048 >> 4)), idesc_pv,
                                  (!first || kk > 0) ? 1u : 0u);
                tc_commit(&bars->pv_done[g][b]);        // the P buffer and the V stage are free
                if (last) tc_commit(&bars->o_full[g]);
            }
            __syncwarp();
            return true;
        };
        while (ok) {
            // the row's entry from the producer (rows without blocks never get here)
            const int slot = i_no & (kPipeRows - 1);
            ok = __all_sync(0xffffffffu, mbar_wait(&bars->row_full[g][slot], (uint32_t)(i_no / kPipeRows) & 1u, abort_flag, p.status)) != 0;
            if (!ok) break;
            const int n = bars->rows[g][slot].z;
            if (n == 0) break;                      // no more rows
            ok = __all_sync(0xffffffffu, mbar_wait(&bars->q_full[g], (uint32_t)i_no & 1u, abort_flag, p.status)) != 0;
            for (int j = 0; ok && j < n; ++j) {
                const int t = t0 + j, b = t & 1;
                ok = __all_sync(0xffffffffu, mbar_wait(&bars->k_full[g][kr.stage], kr.use, abort_flag, p.status)) != 0;
                if (ok) ok = __all_sync(0xffffffffu, mbar_wait(&bars->s_empty[g][b], ((uint32_t)(t >> 1) & 1u) ^ 1u, abort_flag, p.status)) != 0;
                if (!ok) break;
                tc_fence_after();
                const uint64_t db = k_desc + (uint64_t)((kr.stage * kTileBytes) >> 4);
                const uint32_t d = s_tmem + (uint32_t)(64 * b);
                if (elect_one()) {
#pragma unroll
                    for (int kk = 0; kk < kTile / 16; ++kk)
                        tc_mma_f16(d, q_desc + (uint64_t)(kk * 2), db + (uint64_t)(kk * 2), idesc_qk, kk > 0 ? 1u : 0u);
                    tc_commit(&bars->qk_done[g][kr.stage]);     // S is ready and the K stage is free
                    if (j == n - 1) tc_commit(&bars->q_empty[g]);
                }
                __syncwarp();
                kr.next();
                if (j >= 2) ok = issue_pv(t - 2, i_no, j == 2, false);
            }
            for (int j = n < 2 ? 0 : n - 2; ok && j < n; ++j) ok = issue_pv(t0 + j, i_no, j == 0, j == n - 1);
            t0 += n;
            ++i_no;
        }
        // All MMAs issued by the elected lane (the same one every time: the election is deterministic
        // for a converged warp) must have retired before TMEM is freed.
        if (elect_one()) {
            tc_commit(&bars->drain);
            mbar_wait(&bars->drain, 0, abort_flag, p.status);
        }
        __syncwarp();
    } else {
        // ------------------------------------------------------------ softmax warpgroup
        const int quad = warp & 3;                  // TMEM sub-partition this warp may read
        const int q4 = lane & 3;                    // position in the quad: columns 8u + 2 * q4 + {0, 1}
        const int row_a = quad * 16 + (lane >> 2);  // this lane's two rows of the 64-row block
        const uint32_t lane_field = (uint32_t)(quad * 32) << 16;
        const bool masked_op = MASKED && (p.causal != 0 || p.kpm != nullptr || p.quadrants != 0);
        const float c2 = p.scale_log2, c2abs = fabsf(c2);
        const bool flip = c2 < 0.f;
        int t0 = 0, i_no = 0;                       // tiles and non-empty rows before the current row
        KRing kr;                                   // K stage (= qk_done barrier) of the next tile to be requested from TMEM
        bool ok = true;
        while (ok) {
            // The row's entry from the producer (which walks the work items; rows without blocks never get here).
            // The bookkeeping of a work-item cursor in these warps cost 2 000 cycles per row.
            const int slot = i_no & (kPipeRows - 1);
            ok = __all_sync(0xffffffffu, mbar_wait(&bars->row_full[g][slot], (uint32_t)(i_no / kPipeRows) & 1u, abort_flag, p.status)) != 0;
            if (!ok) break;
            const int4 row = bars->rows[g][slot];
            const int n = row.z;
            if (n == 0) break;                      // no more rows
            const size_t lse_a = (size_t)row.x * p.seq_q + (size_t)row.y * kTile + row_a;
            const size_t o_row_a = lse_a * kTile;
            const size_t o_row_b = o_row_a + (size_t)8 * kTile;
            {
                const uint8_t* kpm_row = p.kpm ? p.kpm + (size_t)(row.x / p.kpm_div) * p.kpm_stride : nullptr;
                const int qpos_a = row.y * kTile + row_a;
                // Bits 0-15: columns (u, e) of row a that are masked in block `col`; bits 16-31: row b.
                auto block_mask = [&](const BlockDesc& desc) -> uint32_t {
                    const int col = desc.col();
                    uint32_t m = 0;
                    if (p.quadrants) {
                        // this lane's rows lie in row half quad / 2; its columns 8u + .. in column half u / 4
                        const uint32_t present = (uint32_t)desc.idx >> (2 * (quad >> 1));
                        if (!(present & 1u)) m |= 0x00FF00FFu;
                        if (!(present & 2u)) m |= 0xFF00FF00u;
                    }
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
                // One pass over the row's blocks with a running row maximum m (in units of log2:
                // t = scale * log2(e) * s).  P_j = exp2(t_j - m) goes to tensor memory as the A operand of
                // O += P_j V_j, l sums the P's.  m is only raised when a block's maximum exceeds it by more
                // than kSlack (P stays <= 2^kSlack, exact in fp32 sums and well inside the 16-bit range);
                // raising it rescales O in TMEM and l by exp2(m_old - m_new), which needs the previous
                // P V to have retired.
                constexpr float kSlack = 8.f;
                float m_a = -INFINITY, m_b = -INFINITY;
                // row sums: per row four independent accumulators (even / odd column units x the two columns of a pair)
                float la[4] = {0.f, 0.f, 0.f, 0.f}, lb[4] = {0.f, 0.f, 0.f, 0.f};
                uint32_t r[32];
                // wait for S of tile t (K stage / barrier position kr), unless an earlier test has seen it
                // complete, and start loading it
                auto request_s = [&](int t, bool seen) -> bool {
                    if (!__all_sync(0xffffffffu, seen) &&
                        !__all_sync(0xffffffffu, mbar_wait(&bars->qk_done[g][kr.stage], kr.use, abort_flag, p.status))) return false;
                    kr.next();
                    tc_fence_after();
                    tc_ld_16x256b_x8(s_tmem + lane_field + (uint32_t)(64 * (t & 1)), r);
                    return true;
                };
                bool s_seen = false;                // an earlier test has seen S of the next tile complete
                for (int j = 0; ok && j < n; ++j) {
                    const int t = t0 + j, b = t & 1;
                    ok = request_s(t, s_seen);
                    if (!ok) break;
                    // (the mask of a block is computed while its S tile is on the way)
                    uint32_t mask = 0u;
                    if (MASKED && masked_op) mask = block_mask(bars->descs[g][t & (kPipeDescs - 1)]);
                    tc_wait_ld();
                    release_accumulator(&bars->s_empty[g][b], lane);       // S is in registers: its buffer may be overwritten
                    // Is the P buffer free (P V of tile t - 2 retired), is S of the next tile ready (Q K^T runs two
                    // tiles ahead)?  Tested now, needed after the arithmetic: a test of a barrier costs a few hundred
                    // cycles of latency even when the phase completed long ago.
                    const bool p_free = t < 2 || mbar_test(&bars->pv_done[g][b], ((uint32_t)(t >> 1) & 1u) ^ 1u);
                    s_seen = j + 1 < n && mbar_test(&bars->qk_done[g][kr.stage], kr.use);
                    // Masked elements (above the diagonal, padded keys, quadrants outside a block-32 layout) are
                    // overwritten by -inf (+inf for a negative scale): they lose every maximum and their exp2 is
                    // exactly 0 (the host keeps the scale factor away from 0, so inf * scale is never NaN).
                    if (MASKED && masked_op && mask != 0u) {
                        const uint32_t gone = flip ? 0x7F800000u : 0xFF800000u;
#pragma unroll
                        for (int i = 0; i < 16; ++i) {
                            const int u = i >> 1, e = i & 1;
                            if ((mask >> i) & 1u) r[4 * u + e] = gone;
                            if ((mask >> (16 + i)) & 1u) r[4 * u + 2 + e] = gone;
                        }
                    }
                    // block maxima of the raw scores (for a negative scale: of their negatives), two chains per row
                    float x_a, x_b;
                    {
                        float a0, a1, b0, b1;
                        if (!flip) {
                            a0 = a1 = b0 = b1 = -INFINITY;
#pragma unroll
                            for (int u = 0; u < 8; u += 2) {
                                a0 = fmax3(a0, __uint_as_float(r[4 * u]), __uint_as_float(r[4 * u + 1]));
                                b0 = fmax3(b0, __uint_as_float(r[4 * u + 2]), __uint_as_float(r[4 * u + 3]));
                                a1 = fmax3(a1, __uint_as_float(r[4 * u + 4]), __uint_as_float(r[4 * u + 5]));
                                b1 = fmax3(b1, __uint_as_float(r[4 * u + 6]), __uint_as_float(r[4 * u + 7]));
                            }
                            x_a = fmaxf(a0, a1); x_b = fmaxf(b0, b1);
                        } else {
                            a0 = a1 = b0 = b1 = INFINITY;
#pragma unroll
                            for (int u = 0; u < 8; u += 2) {
                                a0 = fmin3(a0, __uint_as_float(r[4 * u]), __uint_as_float(r[4 * u + 1]));
                                b0 = fmin3(b0, __uint_as_float(r[4 * u + 2]), __uint_as_float(r[4 * u + 3]));
                                a1 = fmin3(a1, __uint_as_float(r[4 * u + 4]), __uint_as_float(r[4 * u + 5]));
                                b1 = fmin3(b1, __uint_as_float(r[4 * u + 6]), __uint_as_float(r[4 * u + 7]));
                            }
                            x_a = -fminf(a0, a1); x_b = -fminf(b0, b1);
                        }
                    }
                    x_a = fmaxf(x_a, __shfl_xor_sync(0xffffffffu, x_a, 1)); x_a = fmaxf(x_a, __shfl_xor_sync(0xffffffffu, x_a, 2));
                    x_b = fmaxf(x_b, __shfl_xor_sync(0xffffffffu, x_b, 1)); x_b = fmaxf(x_b, __shfl_xor_sync(0xffffffffu, x_b, 2));
                    x_a = x_a == -INFINITY ? -INFINITY : x_a * c2abs;       // maxima of t over the block
                    x_b = x_b == -INFINITY ? -INFINITY : x_b * c2abs;
                    if (j == 0) {
                        m_a = x_a; m_b = x_b;                                 // the row's first P V overwrites O
                    } else {
                        // raise a row's maximum only when it is overdue (or was -inf: nothing kept yet)
                        const bool up_a = x_a > m_a + kSlack || (m_a == -INFINITY && x_a > -INFINITY);
                        const bool up_b = x_b > m_b + kSlack || (m_b == -INFINITY && x_b > -INFINITY);
                        if (__any_sync(0xffffffffu, up_a || up_b)) {
                            const float al_a = !up_a ? 1.f : (m_a == -INFINITY ? 0.f : attn_exp2(m_a - x_a));
                            const float al_b = !up_b ? 1.f : (m_b == -INFINITY ? 0.f : attn_exp2(m_b - x_b));
                            if (up_a) { m_a = x_a; la[0] *= al_a; la[1] *= al_a; la[2] *= al_a; la[3] *= al_a; }
                            if (up_b) { m_b = x_b; lb[0] *= al_b; lb[1] *= al_b; lb[2] *= al_b; lb[3] *= al_b; }
                            // O is complete up to the previous tile once that tile's P V has retired
                            if (!__all_sync(0xffffffffu, mbar_wait(&bars->pv_done[g][(t - 1) & 1], (uint32_t)((t - 1) >> 1) & 1u, abort_flag, p.status))) { ok = false; break; }
                            tc_fence_after();
                            for (int c = 0; c < kTile; c += 16) {
                                uint32_t o[8];
                                tc_ld_16x256b_x2(o_tmem + lane_field + (uint32_t)c, o);
                                tc_wait_ld();
#pragma unroll
                                for (int u = 0; u < 2; ++u) {
                                    o[4 * u] = __float_as_uint(__uint_as_float(o[4 * u]) * al_a);
                                    o[4 * u + 1] = __float_as_uint(__uint_as_float(o[4 * u + 1]) * al_a);
                                    o[4 * u + 2] = __float_as_uint(__uint_as_float(o[4 * u + 2]) * al_b);
                                    o[4 * u + 3] = __float_as_uint(__uint_as_float(o[4 * u + 3]) * al_b);
                                }
                                tc_st_16x256b_x2(o_tmem + lane_field + (uint32_t)c, o);
                            }
                            tc_wait_st();
                            tc_fence_before();      // ordered before the P V this block's arrival releases
                        }
                    }
                    const float sub_a = m_a == -INFINITY ? 0.f : m_a, sub_b = m_b == -INFINITY ? 0.f : m_b;
                    // P = exp2(c2 * s - m): per element one FMA, one exp2, one add into the row sum, per pair one pack.
                    // (Scalar instructions: the two-wide fp32 forms save a third of the arithmetic instructions but
                    // need their operands in aligned register pairs, and the moves that arrange them cost more than
                    // they save here: 0.109 against 0.106 ms.)  w[2u + h]: columns 8u + 2 q4 + {0, 1} of row a (h = 0) /
                    // row b (h = 1): the register order of the 16x128b store.
                    uint32_t w[16];
#pragma unroll
                    for (int u = 0; u < 8; ++u) {
#pragma unroll
                        for (int h = 0; h < 2; ++h) {
                            float e0 = fmaf(__uint_as_float(r[4 * u + 2 * h]), c2, h ? -sub_b : -sub_a);
                            float e1 = fmaf(__uint_as_float(r[4 * u + 2 * h + 1]), c2, h ? -sub_b : -sub_a);
                            e0 = attn_exp2(e0); e1 = attn_exp2(e1);
                            if (h) { lb[2 * (u & 1)] += e0; lb[2 * (u & 1) + 1] += e1; }
                            else   { la[2 * (u & 1)] += e0; la[2 * (u & 1) + 1] += e1; }
                            w[2 * u + h] = pack2<BF16>(e0, e1);
                        }
                    }
                    // the P buffer must have been read by the MMAs that used it last (those of tile t - 2)
                    if (!__all_sync(0xffffffffu, p_free) &&
                        !__all_sync(0xffffffffu, mbar_wait(&bars->pv_done[g][b], ((uint32_t)(t >> 1) & 1u) ^ 1u, abort_flag, p.status))) { ok = false; break; }
                    tc_fence_after();
                    tc_st_16x128b_x8(p_tmem + lane_field + (uint32_t)(32 * b), w);
                    tc_wait_st();
                    tc_fence_before();
                    __syncwarp();
                    if (lane == 0) mbar_arrive(&bars->p_full[g][b]);
                }
                t0 += n;
                if (!ok) break;
                // ---- end of the row: O / l and the log-sum-exp
                float l_a, l_b;
                {
                    l_a = (la[0] + la[1]) + (la[2] + la[3]);
                    l_b = (lb[0] + lb[1]) + (lb[2] + lb[3]);
                }
                l_a += __shfl_xor_sync(0xffffffffu, l_a, 1); l_a += __shfl_xor_sync(0xffffffffu, l_a, 2);
                l_b += __shfl_xor_sync(0xffffffffu, l_b, 1); l_b += __shfl_xor_sync(0xffffffffu, l_b, 2);
                const float inv_a = l_a > 0.f ? __frcp_rn(l_a) : 0.f, inv_b = l_b > 0.f ? __frcp_rn(l_b) : 0.f;
                ok = __all_sync(0xffffffffu, mbar_wait(&bars->o_full[g], (uint32_t)i_no & 1u, abort_flag, p.status)) != 0;
                if (!ok) break;
                tc_fence_after();
                uint32_t acc[2][16];
                tc_ld_16x256b_x4(o_tmem + lane_field, acc[0]);
                tc_ld_16x256b_x4(o_tmem + lane_field + 32u, acc[1]);
                tc_wait_ld();
                release_accumulator(&bars->o_empty[g], lane);          // the next row's P V may overwrite O
#pragma unroll
                for (int hc = 0; hc < 2; ++hc) {
                    uint32_t ta[4], tb[4];
#pragma unroll
                    for (int u = 0; u < 4; ++u) {
                        // a row without an unmasked score gets zeros whatever its accumulator holds
                        ta[u] = pack2<BF16>(inv_a > 0.f ? __uint_as_float(acc[hc][4 * u]) * inv_a : 0.f,
                                            inv_a > 0.f ? __uint_as_float(acc[hc][4 * u + 1]) * inv_a : 0.f);
                        tb[u] = pack2<BF16>(inv_b > 0.f ? __uint_as_float(acc[hc][4 * u + 2]) * inv_b : 0.f,
                                            inv_b > 0.f ? __uint_as_float(acc[hc][4 * u + 3]) * inv_b : 0.f);
                    }
                    quad_transpose(ta, q4);         // now columns 32 hc + 8 * q4 .. + 7 of the row
                    quad_transpose(tb, q4);
                    *reinterpret_cast<uint4*>(p.o + o_row_a + 32 * hc + 8 * q4) = make_uint4(ta[0], ta[1], ta[2], ta[3]);
                    *reinterpret_cast<uint4*>(p.o + o_row_b + 32 * hc + 8 * q4) = make_uint4(tb[0], tb[1], tb[2], tb[3]);
                }
                if (q4 == 0 && p.lse) {
                    // natural-log sum of exponentials of the scaled, masked scores
                    p.lse[lse_a] = l_a > 0.f ? (m_a + __log2f(l_a)) * 0.6931471805599453f : -INFINITY;
                    p.lse[lse_a + 8] = l_b > 0.f ? (m_b + __log2f(l_b)) * 0.6931471805599453f : -INFINITY;
                }
                ++i_no;
            }
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
                      const uint8_t* kpm, int64_t kpm_batches, int64_t kpm_stride, int quadrants, uint32_t* workspace,
                      cudaStream_t stream) {
    using KernelFn = void (*)(const CUtensorMap, const CUtensorMap, const CUtensorMap, const AttnParams);
    const bool masked = causal != 0 || kpm != nullptr || quadrants != 0;
    // head dim 64: two independent pipelines per CTA; head dim 128: one softmax warpgroup per CTA
    const bool pipes = head_dim == 64;
    KernelFn kernel;
    if (dtype == BSA_DTYPE_BF16) {
        if (pipes) kernel = masked ? attention_forward_pipes_kernel<true, true> : attention_forward_pipes_kernel<true, false>;
        else       kernel = masked ? attention_forward_kernel<true, true> : attention_forward_kernel<true, false>;
    } else {
        if (pipes) kernel = masked ? attention_forward_pipes_kernel<false, true> : attention_forward_pipes_kernel<false, false>;
        else       kernel = masked ? attention_forward_kernel<false, true> : attention_forward_kernel<false, false>;
    }
    AttnParams p{};
    p.dtiles = (int)(head_dim / kTile);
    p.ring = p.dtiles == 1 ? 4 : 2;
    p.ring_shift = p.dtiles == 1 ? 2 : 1;
    p.vring = p.dtiles == 1 ? 4 : 2;
    p.vring_shift = p.dtiles == 1 ? 2 : 1;
    // at least 80 KB, so that never more than two CTAs (256 TMEM columns each) share an SM
    p.qbufs = p.dtiles == 1 ? 2 : 1;
    int smem_bytes = pipes ? 1024 + 2 * kPipeTiles * kTileBytes + (int)sizeof(PipeBarriers)
                           : 1024 + ((p.qbufs + p.ring + p.vring) * p.dtiles + 2) * kTileBytes + (int)sizeof(AttnBarriers);
    if (smem_bytes < 80 * 1024) smem_bytes = 80 * 1024;
    if (!ensure_dynamic_smem(reinterpret_cast<const void*>(kernel), smem_bytes)) return BSA_ERR_LAUNCH;
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
    if (p.scale_log2 == 0.f) p.scale_log2 = 1e-30f;      // all scores equal, and inf * scale_log2 stays inf for masked ones
    p.causal = causal;
    p.quadrants = quadrants;
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
    // walkers of the work-item list: the CTAs, or (head dim 64) the two pipelines of every CTA
    const int wanted = pipes ? (p.items + 1) / 2 : p.items;
    const unsigned grid = (unsigned)(wanted < 2 * sms ? wanted : 2 * sms);
    const int walkers = pipes ? 2 * (int)grid : (int)grid;
    p.stride_z = walkers / p.groups;
    p.stride_rem = walkers % p.groups;
    kernel<<<grid, (pipes ? 12 : 8) * 32, smem_bytes, stream>>>(map_q, map_k, map_v, p);
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
                                     int quadrant_masks, void* workspace, size_t workspace_bytes, void* stream) {
    using namespace bsa;
    if (dtype != BSA_DTYPE_F32 && dtype != BSA_DTYPE_F16 && dtype != BSA_DTYPE_BF16) return BSA_ERR_BAD_DTYPE;
    if (!valid_block(block)) return BSA_ERR_BAD_BLOCK;
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
                             head_dim, scale, causal, key_padding_mask, kpm_batches, kpm_stride, quadrant_masks != 0,
                             static_cast<uint32_t*>(workspace), static_cast<cudaStream_t>(stream));
}
