// Shared declarations of the block-sparse attention kernel library.
#pragma once

#include <cuda.h>
#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include "bsa.h"

namespace bsa {

// One entry of a layout's `blocks` array: the wire format the reference
// defines in sparse/layout.py:22-26 and reads in sparse/native/sparse_layout.cuh:13-21.
// The reference decodes the column with `& 0xFF`; the packing holds 16 bits.
struct BlockDesc {
    int32_t idx;
    int32_t packed;
    __host__ __device__ __forceinline__ int row() const { return (int)(((uint32_t)packed) >> 16); }
    __host__ __device__ __forceinline__ int col() const { return (int)(((uint32_t)packed) & 0xFFFFu); }
};
static_assert(sizeof(BlockDesc) == 8, "BlockDesc must match the int32 pair wire format");

__host__ __device__ __forceinline__ int dtype_bytes(int dtype) {
    return dtype == BSA_DTYPE_F32 ? 4 : 2;
}

template <typename T> struct Scalar;
template <> struct Scalar<float> {
    static __device__ __forceinline__ float to_float(float v) { return v; }
    static __device__ __forceinline__ float from_float(float v) { return v; }
};
template <> struct Scalar<__half> {
    static __device__ __forceinline__ float to_float(__half v) { return __half2float(v); }
    static __device__ __forceinline__ __half from_float(float v) { return __float2half_rn(v); }
};
template <> struct Scalar<__nv_bfloat16> {
    static __device__ __forceinline__ float to_float(__nv_bfloat16 v) { return __bfloat162float(v); }
    static __device__ __forceinline__ __nv_bfloat16 from_float(float v) { return __float2bfloat16_rn(v); }
};

inline bool aligned16(const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15u) == 0; }
inline bool valid_block(int block) { return block == 16 || block == 32 || block == 64 || block == 128; }

// Turns the sticky/last CUDA error after a launch into a status code.
inline int launch_status() {
    cudaError_t e = cudaGetLastError();
    return e == cudaSuccess ? BSA_OK : BSA_ERR_LAUNCH;
}

// ---- internal entry points of the two matmul engines ---------------------
struct MatmulArgs {
    int mode, dtype, trans_a, trans_b;
    const void* a;
    const void* b;
    void* c;
    const BlockDesc* blocks;
    const int32_t* table;
    int64_t nnz, groups, batches, size_m, size_n, size_k;
    int block;
    uint32_t* workspace;
    cudaStream_t stream;
};

int matmul_simt(const MatmulArgs& args);
// Returns BSA_ERR_BAD_SHAPE etc. on failure; `tc_supports` says whether the
// tcgen05 engine covers a problem at all.
bool tc_supports(const MatmulArgs& args);
int matmul_tc(const MatmulArgs& args);
// The same for the block-32 tcgen05 engine (fp16 / bf16, and fp32 as a 3xTF32 split).
bool tc32_supports(const MatmulArgs& args);
int matmul_tc32(const MatmulArgs& args);
// fused attention kernels: supported dtype / head dim / block combinations
bool attention_supports(int dtype, int64_t head_dim, int block);

}  // namespace bsa
