// Block-sparse row softmax, forward and backward.
//
// Semantics follow the reference kernels sparse_softmax_32x32_forward_kernel
// (sparse_softmax.cu:113-155) and ..._backward_kernel (:165-205): every dense
// row is normalised over the elements of the nonzero blocks of its block row.
// The reference makes 4 reads + 2 writes (forward) and 5 reads + 2 writes
// (backward) per element; here a row is held in registers, so the forward
// moves 1 read + 1 write and the backward 2 reads + 1 write per element,
// all as 128-bit accesses.  Scale, causal and key-padding masks are fused.
//
// Work decomposition: one CTA per (batch, block row).  A dense row of that
// block row is n_blocks segments of `block` contiguous elements, i.e.
// n_blocks * CPS 16-byte chunks.  A team of L lanes (L a power of two,
// 1..256, uniform per CTA) owns one row; lane t holds chunks t, t+L, ...
// (at most kMaxChunks).  Teams narrower than a warp reduce with xor
// shuffles, wider ones add one shared-memory exchange.  Block rows too long
// for registers take a streaming three-pass path.
#include <math_constants.h>

#include <algorithm>

#include "bsa_common.cuh"

namespace bsa {
namespace {

constexpr int kThreads = 256;
constexpr int kWarps = kThreads / 32;
constexpr int kMaxChunks = 8;             // 16-byte chunks a lane keeps in registers
constexpr int kMaxRowBlocksSmem = 2048;   // descriptors staged in shared memory
constexpr float kLog2e = 1.4426950408889634f;

template <typename T> struct Vec;
template <> struct Vec<float> {
    static constexpr int N = 4;
    static __device__ __forceinline__ void load(const float* p, float (&v)[4]) {
        const float4 r = *reinterpret_cast<const float4*>(p);
        v[0] = r.x; v[1] = r.y; v[2] = r.z; v[3] = r.w;
    }
    static __device__ __forceinline__ void unpack(const uint4& r, float (&v)[4]) {
        v[0] = __uint_as_float(r.x); v[1] = __uint_as_float(r.y); v[2] = __uint_as_float(r.z); v[3] = __uint_as_float(r.w);
    }
    static __device__ __forceinline__ void store(float* p, const float (&v)[4]) {
        *reinterpret_cast<float4*>(p) = make_float4(v[0], v[1], v[2], v[3]);
    }
};
template <> struct Vec<__half> {
    static constexpr int N = 8;
    static __device__ __forceinline__ void load(const __half* p, float (&v)[8]) {
        const uint4 r = *reinterpret_cast<const uint4*>(p);
        const __half2* h = reinterpret_cast<const __half2*>(&r);
#pragma unroll
        for (int i = 0; i < 4; ++i) { const float2 f = __half22float2(h[i]); v[2 * i] = f.x; v[2 * i + 1] = f.y; }
    }
    static __device__ __forceinline__ void unpack(const uint4& r, float (&v)[8]) {
        const __half2* h = reinterpret_cast<const __half2*>(&r);
#pragma unroll
        for (int i = 0; i < 4; ++i) { const float2 f = __half22float2(h[i]); v[2 * i] = f.x; v[2 * i + 1] = f.y; }
    }
    static __device__ __forceinline__ void store(__half* p, const float (&v)[8]) {
        uint4 r;
        __half2* h = reinterpret_cast<__half2*>(&r);
#pragma unroll
        for (int i = 0; i < 4; ++i) h[i] = __floats2half2_rn(v[2 * i], v[2 * i + 1]);
        *reinterpret_cast<uint4*>(p) = r;
    }
};
template <> struct Vec<__nv_bfloat16> {
    static constexpr int N = 8;
    static __device__ __forceinline__ void load(const __nv_bfloat16* p, float (&v)[8]) {
        const uint4 r = *reinterpret_cast<const uint4*>(p);
        const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&r);
#pragma unroll
        for (int i = 0; i < 4; ++i) { const float2 f = __bfloat1622float2(h[i]); v[2 * i] = f.x; v[2 * i + 1] = f.y; }
    }
    static __device__ __forceinline__ void unpack(const uint4& r, float (&v)[8]) {
        const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&r);
#pragma unroll
        for (int i = 0; i < 4; ++i) { const float2 f = __bfloat1622float2(h[i]); v[2 * i] = f.x; v[2 * i + 1] = f.y; }
    }
    static __device__ __forceinline__ void store(__nv_bfloat16* p, const float (&v)[8]) {
        uint4 r;
        __nv_bfloat162* h = reinterpret_cast<__nv_bfloat162*>(&r);
#pragma unroll
        for (int i = 0; i < 4; ++i) h[i] = __floats2bfloat162_rn(v[2 * i], v[2 * i + 1]);
        *reinterpret_cast<uint4*>(p) = r;
    }
};

struct SoftmaxParams {
    const void* in0;   // forward: x          backward: y
    const void* in1;   // forward: unused     backward: dy
    void* out;         // forward: y          backward: dx
    const BlockDesc* row_blocks;
    const int32_t* row_table;
    int64_t nnz;
    int block_rows;
    int block;
    float scale;
    int causal;
    const uint8_t* kpm;
    int64_t kpm_stride;
    int64_t batches_per_kpm;
    int skip_upto_chunks;   // general kernel: rows this short were done by the fast kernel
};

// Reduce over a team of L lanes.  For L <= 32 the team lies inside one warp.
// For L > 32 it is L/32 consecutive warps and `exchange` (kWarps floats) is
// used; every thread of the CTA must call this the same number of times.
template <bool kIsMax>
__device__ __forceinline__ float team_reduce(float v, int L, float* exchange) {
    if (L >= 32) {                                // uniform per CTA: the whole warp, unrolled
#pragma unroll
        for (int d = 16; d > 0; d >>= 1) {
            const float o = __shfl_xor_sync(0xffffffffu, v, d);
            v = kIsMax ? fmaxf(v, o) : v + o;
        }
    } else {
        for (int d = L >> 1; d > 0; d >>= 1) {
            const float o = __shfl_xor_sync(0xffffffffu, v, d);
            v = kIsMax ? fmaxf(v, o) : v + o;
        }
    }
    if (L > 32) {
        const int warp = threadIdx.x >> 5;
        if ((threadIdx.x & 31) == 0) exchange[warp] = v;
        __syncthreads();
        const int wpt = L >> 5;
        const int first = (warp / wpt) * wpt;
        v = exchange[first];
        for (int w = 1; w < wpt; ++w) v = kIsMax ? fmaxf(v, exchange[first + w]) : v + exchange[first + w];
    }
    return v;
}

// 2^x by the special-function unit (relative error about 2^-22; 2^-inf = 0).
__device__ __forceinline__ float fast_exp2(float x) {
    float y;
    asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
    return y;
}

// 1 / x by the special-function unit (1 ulp).
__device__ __forceinline__ float fast_rcp(float x) {
    float y;
    asm("rcp.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
    return y;
}

// Scale the logits of one chunk into the log2 domain and mask them.
template <int N>
__device__ __forceinline__ void scale_and_mask(float (&v)[N], float scale_log2e, int q_pos, int k_pos0,
                                               bool causal, const uint8_t* kpm_row) {
#pragma unroll
    for (int e = 0; e < N; ++e) {
        float s = v[e] * scale_log2e;
        if (causal && k_pos0 + e > q_pos) s = -CUDART_INF_F;
        if (kpm_row != nullptr && kpm_row[k_pos0 + e] != 0) s = -CUDART_INF_F;
        v[e] = s;
    }
}

// Bit e set = element e of a chunk lies above the diagonal (key position > query position).
template <int N>
__device__ __forceinline__ uint32_t causal_bits(int q_pos, int k_pos0) {
    constexpr uint32_t full = (1u << N) - 1u;
    const int d = q_pos - k_pos0;                       // elements 0 .. d are visible
    const uint32_t keep = d < 0 ? 0u : (d >= N - 1 ? full : ((2u << d) - 1u));
    return full & ~keep;
}

template <typename T, bool kBackward>
__global__ void __launch_bounds__(kThreads)
softmax_kernel(const SoftmaxParams p) {
    constexpr int N = Vec<T>::N;
    __shared__ BlockDesc s_desc[kMaxRowBlocksSmem];
    __shared__ float s_red0[kWarps], s_red1[kWarps];

    const int block = p.block;
    const int cps = block / N;                    // chunks per segment
    const int r = blockIdx.x;                     // block row
    const int64_t z = blockIdx.y;                 // flattened batch * head
    const int first = p.row_table[r];
    const int n_blocks = p.row_table[r + 1] - first;
    if (n_blocks <= 0) return;                    // uniform for the CTA
    const int n_chunks = n_blocks * cps;
    if (n_chunks <= p.skip_upto_chunks) return;

    for (int j = threadIdx.x; j < n_blocks && j < kMaxRowBlocksSmem; j += kThreads)
        s_desc[j] = p.row_blocks[first + j];
    __syncthreads();

    const T* in0 = static_cast<const T*>(p.in0) + z * p.nnz * block * block;
    const T* in1 = kBackward ? static_cast<const T*>(p.in1) + z * p.nnz * block * block : nullptr;
    T* out = static_cast<T*>(p.out) + z * p.nnz * block * block;
    const uint8_t* kpm_row = (!kBackward && p.kpm) ? p.kpm + (z / p.batches_per_kpm) * p.kpm_stride : nullptr;
    const float scale_log2e = p.scale * kLog2e;
    const bool causal = !kBackward && p.causal != 0;

    // team width: smallest power of two with L * kMaxChunks >= n_chunks
    int L = 1;
    while (L * kMaxChunks < n_chunks && L < kThreads) L <<= 1;

    if (L * kMaxChunks >= n_chunks) {
        // ---------------- register-resident path ----------------
        const int team = threadIdx.x / L, t = threadIdx.x % L;
        const int rows_per_pass = kThreads / L;
        for (int i0 = 0; i0 < block; i0 += rows_per_pass) {
            const int i = i0 + team;
            const bool active = i < block;
            float v[kMaxChunks][N];
            float w[kBackward ? kMaxChunks : 1][N];
            size_t off[kMaxChunks];
            float acc = kBackward ? 0.f : -CUDART_INF_F;
#pragma unroll
            for (int k = 0; k < kMaxChunks; ++k) {
                const int q = t + k * L;
                if (active && q < n_chunks) {
                    const int j = q / cps, s = q - j * cps;
                    const BlockDesc d = s_desc[j];
                    off[k] = ((size_t)d.idx * block + i) * block + s * N;
                    Vec<T>::load(in0 + off[k], v[k]);
                    if (kBackward) {
                        Vec<T>::load(in1 + off[k], w[k]);
#pragma unroll
                        for (int e = 0; e < N; ++e) acc += v[k][e] * w[k][e];
                    } else {
                        scale_and_mask<N>(v[k], scale_log2e, r * block + i, d.col() * block + s * N, causal, kpm_row);
#pragma unroll
                        for (int e = 0; e < N; ++e) acc = fmaxf(acc, v[k][e]);
                    }
                }
            }
            if (kBackward) {
                const float dot = team_reduce<false>(acc, L, s_red0);
#pragma unroll
                for (int k = 0; k < kMaxChunks; ++k) {
                    const int q = t + k * L;
                    if (active && q < n_chunks) {
                        float o[N];
#pragma unroll
                        for (int e = 0; e < N; ++e) o[e] = p.scale * v[k][e] * (w[k][e] - dot);
                        Vec<T>::store(out + off[k], o);
                    }
                }
                if (L > 32) __syncthreads();   // s_red0 is rewritten by the next pass
            } else {
                float mx = team_reduce<true>(acc, L, s_red0);
                if (mx == -CUDART_INF_F) mx = 0.f;   // fully masked row: exp2(-inf) = 0 below
                float sum = 0.f;
#pragma unroll
                for (int k = 0; k < kMaxChunks; ++k) {
                    const int q = t + k * L;
                    if (active && q < n_chunks) {
#pragma unroll
                        for (int e = 0; e < N; ++e) { v[k][e] = exp2f(v[k][e] - mx); sum += v[k][e]; }
                    }
                }
                sum = team_reduce<false>(sum, L, s_red1);
                const float inv = sum > 0.f ? 1.f / sum : 0.f;
#pragma unroll
                for (int k = 0; k < kMaxChunks; ++k) {
                    const int q = t + k * L;
                    if (active && q < n_chunks) {
#pragma unroll
                        for (int e = 0; e < N; ++e) v[k][e] *= inv;
                        Vec<T>::store(out + off[k], v[k]);
                    }
                }
            }
        }
        return;
    }

    // ---------------- streaming path: the whole CTA walks one row at a time,
    // re-reading it for each pass (rows longer than 2048 chunks) -------------
    for (int i = 0; i < block; ++i) {
        float acc = kBackward ? 0.f : -CUDART_INF_F;
        for (int q = threadIdx.x; q < n_chunks; q += kThreads) {
            const int j = q / cps, s = q - j * cps;
            const BlockDesc d = j < kMaxRowBlocksSmem ? s_desc[j] : p.row_blocks[first + j];
            const size_t o = ((size_t)d.idx * block + i) * block + s * N;
            float a[N];
            Vec<T>::load(in0 + o, a);
            if (kBackward) {
                float b[N];
                Vec<T>::load(in1 + o, b);
#pragma unroll
                for (int e = 0; e < N; ++e) acc += a[e] * b[e];
            } else {
                scale_and_mask<N>(a, scale_log2e, r * block + i, d.col() * block + s * N, causal, kpm_row);
#pragma unroll
                for (int e = 0; e < N; ++e) acc = fmaxf(acc, a[e]);
            }
        }
        float first_red = kBackward ? team_reduce<false>(acc, kThreads, s_red0)
                                    : team_reduce<true>(acc, kThreads, s_red0);
        float inv = 0.f;
        if (!kBackward) {
            if (first_red == -CUDART_INF_F) first_red = 0.f;
            float sum = 0.f;
            for (int q = threadIdx.x; q < n_chunks; q += kThreads) {
                const int j = q / cps, s = q - j * cps;
                const BlockDesc d = j < kMaxRowBlocksSmem ? s_desc[j] : p.row_blocks[first + j];
                const size_t o = ((size_t)d.idx * block + i) * block + s * N;
                float a[N];
                Vec<T>::load(in0 + o, a);
                scale_and_mask<N>(a, scale_log2e, r * block + i, d.col() * block + s * N, causal, kpm_row);
#pragma unroll
                for (int e = 0; e < N; ++e) sum += exp2f(a[e] - first_red);
            }
            sum = team_reduce<false>(sum, kThreads, s_red1);
            inv = sum > 0.f ? 1.f / sum : 0.f;
        }
        for (int q = threadIdx.x; q < n_chunks; q += kThreads) {
            const int j = q / cps, s = q - j * cps;
            const BlockDesc d = j < kMaxRowBlocksSmem ? s_desc[j] : p.row_blocks[first + j];
            const size_t o = ((size_t)d.idx * block + i) * block + s * N;
            float a[N], res[N];
            Vec<T>::load(in0 + o, a);
            if (kBackward) {
                float b[N];
                Vec<T>::load(in1 + o, b);
#pragma unroll
                for (int e = 0; e < N; ++e) res[e] = p.scale * a[e] * (b[e] - first_red);
            } else {
                scale_and_mask<N>(a, scale_log2e, r * block + i, d.col() * block + s * N, causal, kpm_row);
#pragma unroll
                for (int e = 0; e < N; ++e) res[e] = exp2f(a[e] - first_red) * inv;
            }
            Vec<T>::store(out + o, res);
        }
        __syncthreads();   // exchange buffers are reused by the next row
    }
}


// Fast path: rows of at most 256 * CH chunks.  A measured copy kernel with exactly this traversal
// (a warp per dense row, 16-byte chunks, no prefetch) reaches 93 % of the HBM copy peak at full
// occupancy, so the kernel is built to stay small: a lane keeps its CH chunks packed in the
// input type (4 registers per chunk) through all three phases -- maximum (taken on the packed
// values for 16-bit types), exponentials (written back packed, so a 16-bit result carries two
// roundings, about 1e-3 relative), normalisation -- and converts on the fly.  The block
// descriptor of each of a lane's chunks is the same for every row of the block row, so it is
// looked up once per CTA.  Longer rows are left to softmax_kernel.
template <typename T> struct Packed;
template <> struct Packed<float> {
    static __device__ __forceinline__ uint4 pack(const float (&v)[4]) {
        return make_uint4(__float_as_uint(v[0]), __float_as_uint(v[1]), __float_as_uint(v[2]), __float_as_uint(v[3]));
    }
    static __device__ __forceinline__ uint4 scaled(const uint4& r, float f) {
        return make_uint4(__float_as_uint(__uint_as_float(r.x) * f), __float_as_uint(__uint_as_float(r.y) * f),
                          __float_as_uint(__uint_as_float(r.z) * f), __float_as_uint(__uint_as_float(r.w) * f));
    }
    // max over the chunk of sign * x
    static __device__ __forceinline__ float signed_max(const uint4& r, bool negate) {
        const float m0 = negate ? fminf(fminf(__uint_as_float(r.x), __uint_as_float(r.y)), fminf(__uint_as_float(r.z), __uint_as_float(r.w)))
                                : fmaxf(fmaxf(__uint_as_float(r.x), __uint_as_float(r.y)), fmaxf(__uint_as_float(r.z), __uint_as_float(r.w)));
        return negate ? -m0 : m0;
    }
};
template <> struct Packed<__half> {
    static __device__ __forceinline__ uint4 pack(const float (&v)[8]) {
        uint4 r;
        __half2* h = reinterpret_cast<__half2*>(&r);
#pragma unroll
        for (int i = 0; i < 4; ++i) h[i] = __floats2half2_rn(v[2 * i], v[2 * i + 1]);
        return r;
    }
    // Exponentials in [0, 1] times 1 / sum, multiplied as packed halves: the factor is rounded to
    // 11 bits first (2^-11 relative, like the product), which keeps the conversion pipe free.
    static __device__ __forceinline__ uint4 scaled(const uint4& r, float f) {
        uint4 o;
        const __half2* h = reinterpret_cast<const __half2*>(&r);
        __half2* q = reinterpret_cast<__half2*>(&o);
        const __half2 f2 = __float2half2_rn(f);
#pragma unroll
        for (int i = 0; i < 4; ++i) q[i] = __hmul2(h[i], f2);
        return o;
    }
    static __device__ __forceinline__ float signed_max(const uint4& r, bool negate) {
        const __half2* h = reinterpret_cast<const __half2*>(&r);
        const __half2 m = negate ? __hmin2(__hmin2(h[0], h[1]), __hmin2(h[2], h[3]))
                                 : __hmax2(__hmax2(h[0], h[1]), __hmax2(h[2], h[3]));
        const float2 f = __half22float2(m);
        return negate ? -fminf(f.x, f.y) : fmaxf(f.x, f.y);
    }
};
template <> struct Packed<__nv_bfloat16> {
    static __device__ __forceinline__ uint4 pack(const float (&v)[8]) {
        uint4 r;
        __nv_bfloat162* h = reinterpret_cast<__nv_bfloat162*>(&r);
#pragma unroll
        for (int i = 0; i < 4; ++i) h[i] = __floats2bfloat162_rn(v[2 * i], v[2 * i + 1]);
        return r;
    }
    static __device__ __forceinline__ uint4 scaled(const uint4& r, float f) {
        float v[8];
        Vec<__nv_bfloat16>::unpack(r, v);
#pragma unroll
        for (int e = 0; e < 8; ++e) v[e] *= f;
        return pack(v);
    }
    static __device__ __forceinline__ float signed_max(const uint4& r, bool negate) {
        const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&r);
        const __nv_bfloat162 m = negate ? __hmin2(__hmin2(h[0], h[1]), __hmin2(h[2], h[3]))
                                        : __hmax2(__hmax2(h[0], h[1]), __hmax2(h[2], h[3]));
        const float2 f = __bfloat1622float2(m);
        return negate ? -fminf(f.x, f.y) : fmaxf(f.x, f.y);
    }
};

// team_reduce for R independent values at once: the shuffles of the R butterflies interleave and
// teams wider than a warp pay one barrier for all of them.  `exchange` holds R * kWarps floats.
template <bool kIsMax, int R>
__device__ __forceinline__ void team_reduce_n(float (&v)[R], int L, float* exchange) {
    if (L >= 32) {
#pragma unroll
        for (int d = 16; d > 0; d >>= 1) {
#pragma unroll
            for (int u = 0; u < R; ++u) {
                const float o = __shfl_xor_sync(0xffffffffu, v[u], d);
                v[u] = kIsMax ? fmaxf(v[u], o) : v[u] + o;
            }
        }
    } else {
        for (int d = L >> 1; d > 0; d >>= 1) {
#pragma unroll
            for (int u = 0; u < R; ++u) {
                const float o = __shfl_xor_sync(0xffffffffu, v[u], d);
                v[u] = kIsMax ? fmaxf(v[u], o) : v[u] + o;
            }
        }
    }
    if (L > 32) {
        const int warp = threadIdx.x >> 5;
        if ((threadIdx.x & 31) == 0) {
#pragma unroll
            for (int u = 0; u < R; ++u) exchange[u * kWarps + warp] = v[u];
        }
        __syncthreads();
        const int wpt = L >> 5;
        const int first = (warp / wpt) * wpt;
#pragma unroll
        for (int u = 0; u < R; ++u) {
            float r = exchange[u * kWarps + first];
            for (int w = 1; w < wpt; ++w)
                r = kIsMax ? fmaxf(r, exchange[u * kWarps + first + w]) : r + exchange[u * kWarps + first + w];
            v[u] = r;
        }
    }
}

// Rows a team works on per pass.  A lane keeps RPT * CH chunks in flight; with fewer than about
// four 16-byte loads per lane outstanding, 32-40 resident warps do not cover the HBM latency.
constexpr int rows_per_team(int ch, bool backward, bool masked) {
    return backward ? (ch <= 2 ? 2 : 1) : (ch == 1 ? 4 : ch == 2 ? 2 : (ch == 3 && !masked) ? 2 : 1);
}

template <typename T, int CH, int RPT, bool kBackward, bool kMasked>
__global__ void __launch_bounds__(kThreads, CH == 8 ? ((kBackward || kMasked) ? 2 : 3) : (kBackward ? 4 : 5))
softmax_rows_kernel(const SoftmaxParams p) {
    constexpr int N = Vec<T>::N;
    __shared__ float s_red0[RPT * kWarps], s_red1[RPT * kWarps];

    const int block = p.block;
    const int cps = block / N;                    // chunks per segment (a power of two)
    const int cps_shift = 31 - __clz(cps);
    const int r = blockIdx.x;
    const int64_t z = blockIdx.y;
    const int first = p.row_table[r];
    const int n_blocks = p.row_table[r + 1] - first;
    if (n_blocks <= 0) return;
    const int n_chunks = n_blocks << cps_shift;
    if (n_chunks > kThreads * CH) return;         // left to the general kernel

    int L = 1;
    while (L * CH < n_chunks) L <<= 1;            // <= 256
    const int team = threadIdx.x / L, t = threadIdx.x & (L - 1);
    const int rows_per_pass = kThreads / L;

    const uint8_t* kpm_row = (kMasked && p.kpm) ? p.kpm + (z / p.batches_per_kpm) * p.kpm_stride : nullptr;
    uint32_t base[CH];                            // element offset of the lane's chunk in row 0, or ~0
    int kpos[kMasked ? CH : 1];                   // key position of the chunk's first element
    uint32_t kbits[kMasked ? CH : 1];             // bit e: key kpos + e is padding (the same for every row)
#pragma unroll
    for (int k = 0; k < CH; ++k) {
        const int q = t + k * L;
        base[k] = 0xFFFFFFFFu;
        if (kMasked) { kpos[k] = 0; kbits[k] = 0u; }
        if (q < n_chunks) {
            const int j = q >> cps_shift, s = q & (cps - 1);
            const BlockDesc d = p.row_blocks[first + j];
            base[k] = (uint32_t)d.idx * (uint32_t)(block * block) + (uint32_t)(s * N);
            if (kMasked) {
                kpos[k] = d.col() * block + s * N;
                if (kpm_row != nullptr) {
#pragma unroll
                    for (int e = 0; e < N; ++e) kbits[k] |= (kpm_row[kpos[k] + e] != 0 ? 1u : 0u) << e;
                }
            }
        }
    }

    const size_t zoff = (size_t)z * p.nnz * block * block;
    const T* in0 = static_cast<const T*>(p.in0) + zoff;
    const T* in1 = kBackward ? static_cast<const T*>(p.in1) + zoff : nullptr;
    T* out = static_cast<T*>(p.out) + zoff;
    const float scale_log2e = p.scale * kLog2e;
    const bool causal = kMasked && p.causal != 0;
    const bool negate = scale_log2e < 0.f;

    for (int i0 = team; i0 < block; i0 += rows_per_pass * RPT) {
        // row u of this pass is i0 + u * rows_per_pass; rows past the block (short rows, where one
        // pass covers the block) are switched off
        uint4 x[RPT][CH], g[kBackward ? RPT : 1][kBackward ? CH : 1];
        bool on[RPT][CH];
#pragma unroll
        for (int u = 0; u < RPT; ++u) {
            const int i = i0 + u * rows_per_pass;
#pragma unroll
            for (int k = 0; k < CH; ++k) {
                on[u][k] = base[k] != 0xFFFFFFFFu && (u == 0 || i < block);
                if (on[u][k]) {
                    x[u][k] = *reinterpret_cast<const uint4*>(in0 + base[k] + i * block);
                    if (kBackward) g[u][k] = *reinterpret_cast<const uint4*>(in1 + base[k] + i * block);
                }
            }
        }
        if (kBackward) {
            float dot[RPT];
#pragma unroll
            for (int u = 0; u < RPT; ++u) {
                dot[u] = 0.f;
#pragma unroll
                for (int k = 0; k < CH; ++k) {
                    if (on[u][k]) {
                        float v[N], w[N];
                        Vec<T>::unpack(x[u][k], v);
                        Vec<T>::unpack(g[u][k], w);
#pragma unroll
                        for (int e = 0; e < N; ++e) dot[u] = fmaf(v[e], w[e], dot[u]);
                    }
                }
            }
            team_reduce_n<false, RPT>(dot, L, s_red0);
#pragma unroll
            for (int u = 0; u < RPT; ++u) {
                const int i = i0 + u * rows_per_pass;
#pragma unroll
                for (int k = 0; k < CH; ++k) {
                    if (on[u][k]) {
                        float v[N], w[N];
                        Vec<T>::unpack(x[u][k], v);
                        Vec<T>::unpack(g[u][k], w);
#pragma unroll
                        for (int e = 0; e < N; ++e) v[e] = (p.scale * v[e]) * (w[e] - dot[u]);
                        *reinterpret_cast<uint4*>(out + base[k] + i * block) = Packed<T>::pack(v);
                    }
                }
            }
            if (L > 32) __syncthreads();          // s_red0 is rewritten by the next pass
        } else {
            // phase 1: row maximum of scale*log2e*x (masked elements are -inf).  (Sorting chunks into
            // clean / partly masked / fully masked ones to spare the clean ones the element-wise
            // masks was measured slower: the classes diverge inside a warp.)
            float mx[RPT];
#pragma unroll
            for (int u = 0; u < RPT; ++u) {
                const int i = i0 + u * rows_per_pass;
                mx[u] = -CUDART_INF_F;
#pragma unroll
                for (int k = 0; k < CH; ++k) {
                    if (on[u][k]) {
                        if (kMasked) {
                            float v[N];
                            Vec<T>::unpack(x[u][k], v);
                            const uint32_t bits = kbits[kMasked ? k : 0] |
                                                  (causal ? causal_bits<N>(r * block + i, kpos[kMasked ? k : 0]) : 0u);
#pragma unroll
                            for (int e = 0; e < N; ++e)
                                mx[u] = fmaxf(mx[u], ((bits >> e) & 1u) ? -CUDART_INF_F : v[e] * scale_log2e);
                        } else {
                            mx[u] = fmaxf(mx[u], Packed<T>::signed_max(x[u][k], negate));
                        }
                    }
                }
            }
            team_reduce_n<true, RPT>(mx, L, s_red0);
            // phase 2: exponentials (kept packed) and their sum
            float sum[RPT];
#pragma unroll
            for (int u = 0; u < RPT; ++u) {
                const int i = i0 + u * rows_per_pass;
                if (mx[u] == -CUDART_INF_F) mx[u] = 0.f;
                if (!kMasked) mx[u] *= fabsf(scale_log2e);   // max of sign*x -> max of scale*log2e*x
                sum[u] = 0.f;
#pragma unroll
                for (int k = 0; k < CH; ++k) {
                    if (on[u][k]) {
                        float v[N];
                        Vec<T>::unpack(x[u][k], v);
                        if (kMasked) {
                            const uint32_t bits = kbits[kMasked ? k : 0] |
                                                  (causal ? causal_bits<N>(r * block + i, kpos[kMasked ? k : 0]) : 0u);
#pragma unroll
                            for (int e = 0; e < N; ++e)
                                v[e] = ((bits >> e) & 1u) ? 0.f : fast_exp2(fmaf(v[e], scale_log2e, -mx[u]));
                        } else {
#pragma unroll
                            for (int e = 0; e < N; ++e) v[e] = fast_exp2(fmaf(v[e], scale_log2e, -mx[u]));
                        }
#pragma unroll
                        for (int e = 0; e < N; ++e) sum[u] += v[e];
                        x[u][k] = Packed<T>::pack(v);
                    }
                }
            }
            team_reduce_n<false, RPT>(sum, L, s_red1);
            // phase 3: normalise and store
#pragma unroll
            for (int u = 0; u < RPT; ++u) {
                const int i = i0 + u * rows_per_pass;
                const float inv = sum[u] > 0.f ? fast_rcp(sum[u]) : 0.f;
#pragma unroll
                for (int k = 0; k < CH; ++k) {
                    if (on[u][k])
                        *reinterpret_cast<uint4*>(out + base[k] + i * block) = Packed<T>::scaled(x[u][k], inv);
                }
            }
        }
    }
}

int check_common(int dtype, const void* a, const void* b, const void* c,
                 const int32_t* row_blocks, const int32_t* row_table,
                 int64_t nnz, int64_t block_rows, int64_t batches, int block) {
    if (!a || !b || !c || !row_blocks || !row_table) return BSA_ERR_NULL_POINTER;
    if (dtype != BSA_DTYPE_F32 && dtype != BSA_DTYPE_F16 && dtype != BSA_DTYPE_BF16) return BSA_ERR_BAD_DTYPE;
    if (!valid_block(block)) return BSA_ERR_BAD_BLOCK;
    if (nnz < 0 || block_rows <= 0 || batches < 0) return BSA_ERR_BAD_SHAPE;
    if (block_rows > 65535 || batches > 65535 || nnz > (int64_t)INT32_MAX) return BSA_ERR_TOO_LARGE;
    if (!aligned16(a) || !aligned16(b) || !aligned16(c)) return BSA_ERR_ALIGNMENT;
    return BSA_OK;
}

template <typename T, bool kBackward>
int launch_typed(const SoftmaxParams& base, int64_t batches, int64_t max_row_blocks, cudaStream_t stream) {
    SoftmaxParams p = base;
    const dim3 grid((unsigned)p.block_rows, (unsigned)batches);
    const int cps = p.block / Vec<T>::N;
    // chunks per lane: enough for an average row in one warp and, when the longest row is known,
    // for that row in one CTA
    const int64_t avg_chunks = (p.nnz * cps + p.block_rows - 1) / p.block_rows;
    int64_t need = (avg_chunks + 31) / 32;
    if (max_row_blocks > 0) need = std::max<int64_t>(need, (max_row_blocks * cps + kThreads - 1) / kThreads);
    int ch = need <= 1 ? 1 : need <= 2 ? 2 : need <= 3 ? 3 : need <= 4 ? 4 : 8;
    const bool masked = !kBackward && (p.causal != 0 || p.kpm != nullptr);
#define BSA_SOFTMAX_ROWS(CH_)                                                                        \
    if (masked)                                                                                      \
        softmax_rows_kernel<T, CH_, rows_per_team(CH_, kBackward, true), kBackward, !kBackward>      \
            <<<grid, kThreads, 0, stream>>>(p);                                                      \
    else                                                                                             \
        softmax_rows_kernel<T, CH_, rows_per_team(CH_, kBackward, false), kBackward, false>          \
            <<<grid, kThreads, 0, stream>>>(p)
    switch (ch) {
        case 1: BSA_SOFTMAX_ROWS(1); break;
        case 2: BSA_SOFTMAX_ROWS(2); break;
        case 3: BSA_SOFTMAX_ROWS(3); break;
        case 4: BSA_SOFTMAX_ROWS(4); break;
        default: BSA_SOFTMAX_ROWS(8); break;
    }
#undef BSA_SOFTMAX_ROWS
    int st = launch_status();
    if (st != BSA_OK) return st;
    // rows longer than the fast kernel holds (or of unknown length) go to the general kernel
    if (max_row_blocks <= 0 || max_row_blocks * cps > (int64_t)kThreads * ch) {
        p.skip_upto_chunks = kThreads * ch;
        softmax_kernel<T, kBackward><<<grid, kThreads, 0, stream>>>(p);
        st = launch_status();
    }
    return st;
}

template <bool kBackward>
int launch(int dtype, const SoftmaxParams& p, int64_t batches, int64_t max_row_blocks, cudaStream_t stream) {
    if (batches == 0 || p.nnz == 0) return BSA_OK;
    if (p.nnz * (int64_t)p.block * p.block >= ((int64_t)1 << 32)) return BSA_ERR_TOO_LARGE;
    switch (dtype) {
        case BSA_DTYPE_F32: return launch_typed<float, kBackward>(p, batches, max_row_blocks, stream);
        case BSA_DTYPE_F16: return launch_typed<__half, kBackward>(p, batches, max_row_blocks, stream);
        default: return launch_typed<__nv_bfloat16, kBackward>(p, batches, max_row_blocks, stream);
    }
}

}  // namespace
}  // namespace bsa

extern "C" int bsa_softmax_forward(int dtype, const void* x, void* y,
                                   const int32_t* row_blocks, const int32_t* row_table,
                                   int64_t nnz, int64_t block_rows, int64_t batches, int block,
                                   float scale, int causal,
                                   const uint8_t* key_padding_mask, int64_t kpm_batches,
                                   int64_t kpm_stride, int64_t max_row_blocks, void* stream) {
    using namespace bsa;
    int st = check_common(dtype, x, x, y, row_blocks, row_table, nnz, block_rows, batches, block);
    if (st != BSA_OK) return st;
    SoftmaxParams p{};
    p.in0 = x; p.in1 = nullptr; p.out = y;
    p.row_blocks = reinterpret_cast<const BlockDesc*>(row_blocks);
    p.row_table = row_table;
    p.nnz = nnz; p.block_rows = (int)block_rows; p.block = block;
    p.scale = scale; p.causal = causal;
    p.kpm = key_padding_mask; p.kpm_stride = kpm_stride; p.batches_per_kpm = 1;
    if (key_padding_mask) {
        if (kpm_batches <= 0 || batches % kpm_batches != 0 || kpm_stride <= 0) return BSA_ERR_BAD_SHAPE;
        p.batches_per_kpm = batches / kpm_batches;
    }
    return launch<false>(dtype, p, batches, max_row_blocks, static_cast<cudaStream_t>(stream));
}

extern "C" int bsa_softmax_backward(int dtype, const void* y, const void* dy, void* dx,
                                    const int32_t* row_blocks, const int32_t* row_table,
                                    int64_t nnz, int64_t block_rows, int64_t batches, int block,
                                    float scale, int64_t max_row_blocks, void* stream) {
    using namespace bsa;
    int st = check_common(dtype, y, dy, dx, row_blocks, row_table, nnz, block_rows, batches, block);
    if (st != BSA_OK) return st;
    SoftmaxParams p{};
    p.in0 = y; p.in1 = dy; p.out = dx;
    p.row_blocks = reinterpret_cast<const BlockDesc*>(row_blocks);
    p.row_table = row_table;
    p.nnz = nnz; p.block_rows = (int)block_rows; p.block = block;
    p.scale = scale; p.causal = 0;
    p.kpm = nullptr; p.kpm_stride = 0; p.batches_per_kpm = 1;
    return launch<true>(dtype, p, batches, max_row_blocks, static_cast<cudaStream_t>(stream));
}
