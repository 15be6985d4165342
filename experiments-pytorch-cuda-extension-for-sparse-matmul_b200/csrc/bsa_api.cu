// C-ABI entry points that are not tied to one kernel file: version and status
// text, the matmul dispatcher with its argument validation, the dense <->
// block-sparse converters and the workspace status word.
#include <cstdlib>
#include <cstring>
#include <mutex>

#include "bsa_common.cuh"

namespace bsa {
namespace {

// to_sparse / to_dense (reference sparse/layout.py:40-57 are Python loops over
// the nonzero blocks).  One CTA per (block, batch); 16-byte chunks.
template <bool kToSparse>
__global__ void __launch_bounds__(256)
convert_kernel(const uint4* __restrict__ src, uint4* __restrict__ dst, const BlockDesc* __restrict__ row_blocks,
               int64_t nnz, int64_t rows, int64_t cols, int block, int chunks_per_row) {
    const BlockDesc d = row_blocks[blockIdx.x];
    const int64_t z = blockIdx.y;
    const int64_t dense_row_chunks = cols * chunks_per_row;              // chunks in one dense row
    const size_t dense_base = ((size_t)z * rows * block + (size_t)d.row() * block) * dense_row_chunks
                              + (size_t)d.col() * chunks_per_row;
    const size_t sparse_base = ((size_t)z * nnz + d.idx) * block * chunks_per_row;
    for (int t = threadIdx.x; t < block * chunks_per_row; t += blockDim.x) {
        const int i = t / chunks_per_row, c = t - i * chunks_per_row;
        const size_t dn = dense_base + (size_t)i * dense_row_chunks + c;
        if (kToSparse) dst[sparse_base + t] = src[dn];
        else           dst[dn] = src[sparse_base + t];
    }
}

int convert(bool to_sparse, int dtype, const void* src, void* dst, const int32_t* row_blocks,
            int64_t nnz, int64_t batches, int64_t rows, int64_t cols, int block, cudaStream_t stream) {
    if (!src || !dst || !row_blocks) return BSA_ERR_NULL_POINTER;
    if (dtype != BSA_DTYPE_F32 && dtype != BSA_DTYPE_F16 && dtype != BSA_DTYPE_BF16) return BSA_ERR_BAD_DTYPE;
    if (!valid_block(block)) return BSA_ERR_BAD_BLOCK;
    if (nnz < 0 || batches < 0 || rows <= 0 || cols <= 0) return BSA_ERR_BAD_SHAPE;
    if (batches > 65535 || nnz > (int64_t)INT32_MAX) return BSA_ERR_TOO_LARGE;
    if (!aligned16(src) || !aligned16(dst)) return BSA_ERR_ALIGNMENT;
    const int cpr = block * dtype_bytes(dtype) / 16;
    if (!to_sparse) {
        cudaError_t e = cudaMemsetAsync(dst, 0, (size_t)batches * rows * cols * block * block * dtype_bytes(dtype), stream);
        if (e != cudaSuccess) return BSA_ERR_LAUNCH;
    }
    if (nnz == 0 || batches == 0) return BSA_OK;
    const dim3 grid((unsigned)nnz, (unsigned)batches);
    const BlockDesc* rb = reinterpret_cast<const BlockDesc*>(row_blocks);
    if (to_sparse)
        convert_kernel<true><<<grid, 256, 0, stream>>>((const uint4*)src, (uint4*)dst, rb, nnz, rows, cols, block, cpr);
    else
        convert_kernel<false><<<grid, 256, 0, stream>>>((const uint4*)src, (uint4*)dst, rb, nnz, rows, cols, block, cpr);
    return launch_status();
}

}  // namespace
}  // namespace bsa

extern "C" int bsa_version(void) { return 100; /* 0.1.0 */ }

extern "C" const char* bsa_status_string(int status) {
    switch (status) {
        case BSA_OK: return "ok";
        case BSA_ERR_NULL_POINTER: return "a required pointer is NULL";
        case BSA_ERR_BAD_MODE: return "mode must be sdd (0), dsd (1) or dds (2)";
        case BSA_ERR_BAD_DTYPE: return "unsupported dtype";
        case BSA_ERR_BAD_SHAPE: return "bad shape: sizes must be positive and the sparse sides multiples of the block size";
        case BSA_ERR_BAD_BLOCK: return "block size must be 16, 32, 64 or 128";
        case BSA_ERR_ALIGNMENT: return "device pointers must be 16-byte aligned";
        case BSA_ERR_WORKSPACE: return "workspace missing or smaller than BSA_WORKSPACE_BYTES";
        case BSA_ERR_LAUNCH: return "CUDA launch failed";
        case BSA_ERR_DEVICE_TIMEOUT: return "a bounded wait inside a kernel ran out";
        case BSA_ERR_TOO_LARGE: return "a size exceeds the supported maximum";
        case BSA_ERR_DRIVER: return "could not resolve a CUDA driver entry point";
        default: return "unknown status";
    }
}

namespace {
// Host-side argument checks of the matmul entry points; nothing is launched when they fail.
int check_matmul_args(int mode, int dtype, const void* a, const void* b, const void* c,
                      const int32_t* blocks, const int32_t* table, int64_t nnz, int64_t groups, int64_t batches,
                      int64_t size_m, int64_t size_n, int64_t size_k, int block, int engine) {
    if (mode != BSA_MODE_SDD && mode != BSA_MODE_DSD && mode != BSA_MODE_DDS) return BSA_ERR_BAD_MODE;
    if (dtype != BSA_DTYPE_F32 && dtype != BSA_DTYPE_F16 && dtype != BSA_DTYPE_BF16) return BSA_ERR_BAD_DTYPE;
    if (!bsa::valid_block(block)) return BSA_ERR_BAD_BLOCK;
    if (!a || !b || !c || !blocks || !table) return BSA_ERR_NULL_POINTER;
    if (nnz < 0 || groups <= 0 || batches < 0 || size_m <= 0 || size_n <= 0 || size_k <= 0) return BSA_ERR_BAD_SHAPE;
    if (nnz > (int64_t)INT32_MAX / 2 || groups > 65535 || batches > 65535) return BSA_ERR_TOO_LARGE;
    if (engine != BSA_ENGINE_AUTO && engine != BSA_ENGINE_SIMT && engine != BSA_ENGINE_TCGEN05) return BSA_ERR_BAD_MODE;
    // The grouped axis of the sparse operand must match the table.
    const int64_t grouped = groups * block;
    if (mode == BSA_MODE_SDD) {
        // sdd walks the row layout as a flat list: rows of C are the groups.
        if (size_m != grouped || size_n % block != 0) return BSA_ERR_BAD_SHAPE;
    } else if (mode == BSA_MODE_DSD) {
        if (size_m != grouped || size_k % block != 0) return BSA_ERR_BAD_SHAPE;
    } else {
        if (size_n != grouped || size_k % block != 0) return BSA_ERR_BAD_SHAPE;
    }
    if (!bsa::aligned16(a) || !bsa::aligned16(b) || !bsa::aligned16(c)) return BSA_ERR_ALIGNMENT;
    return BSA_OK;
}
}  // namespace

extern "C" int bsa_matmul(int mode, int dtype, int trans_a, int trans_b,
                          const void* a, const void* b, void* c,
                          const int32_t* blocks, const int32_t* table,
                          int64_t nnz, int64_t groups, int64_t batches,
                          int64_t size_m, int64_t size_n, int64_t size_k, int block,
                          void* workspace, size_t workspace_bytes, int engine, void* stream) {
    using namespace bsa;
    // same order of checks as before the split: mode, dtype, block, pointers, workspace, sizes
    if (mode != BSA_MODE_SDD && mode != BSA_MODE_DSD && mode != BSA_MODE_DDS) return BSA_ERR_BAD_MODE;
    if (dtype != BSA_DTYPE_F32 && dtype != BSA_DTYPE_F16 && dtype != BSA_DTYPE_BF16) return BSA_ERR_BAD_DTYPE;
    if (!valid_block(block)) return BSA_ERR_BAD_BLOCK;
    if (!a || !b || !c || !blocks || !table) return BSA_ERR_NULL_POINTER;
    if (!workspace || workspace_bytes < BSA_WORKSPACE_BYTES) return BSA_ERR_WORKSPACE;
    const int checked = check_matmul_args(mode, dtype, a, b, c, blocks, table, nnz, groups, batches,
                                          size_m, size_n, size_k, block, engine);
    if (checked != BSA_OK) return checked;
    if (batches == 0) return BSA_OK;

    MatmulArgs args{mode, dtype, trans_a != 0, trans_b != 0, a, b, c,
                    reinterpret_cast<const BlockDesc*>(blocks), table,
                    nnz, groups, batches, size_m, size_n, size_k, block,
                    static_cast<uint32_t*>(workspace), static_cast<cudaStream_t>(stream)};
    if (engine == BSA_ENGINE_AUTO) {
        const char* env = std::getenv("BSA_MATMUL_ENGINE");
        if (env && std::strcmp(env, "simt") == 0) engine = BSA_ENGINE_SIMT;
        else if (env && std::strcmp(env, "tcgen05") == 0) engine = BSA_ENGINE_TCGEN05;
    }
    if (engine != BSA_ENGINE_SIMT) {
        if (tc_supports(args)) return matmul_tc(args);        // block 64, 16-bit types
        if (tc32_supports(args)) return matmul_tc32(args);    // block 32, 16-bit types and fp32 (3xTF32)
        if (engine == BSA_ENGINE_TCGEN05) return BSA_ERR_BAD_SHAPE;
    }
    return matmul_simt(args);
}

extern "C" int bsa_dense_to_sparse(int dtype, const void* dense, void* sparse,
                                   const int32_t* row_blocks, int64_t nnz, int64_t batches,
                                   int64_t rows, int64_t cols, int block, void* stream) {
    return bsa::convert(true, dtype, dense, sparse, row_blocks, nnz, batches, rows, cols, block,
                        static_cast<cudaStream_t>(stream));
}

extern "C" int bsa_sparse_to_dense(int dtype, const void* sparse, void* dense,
                                   const int32_t* row_blocks, int64_t nnz, int64_t batches,
                                   int64_t rows, int64_t cols, int block, void* stream) {
    return bsa::convert(false, dtype, sparse, dense, row_blocks, nnz, batches, rows, cols, block,
                        static_cast<cudaStream_t>(stream));
}

extern "C" int bsa_workspace_status_detail(void* workspace, void* stream, int32_t* detail) {
    if (detail) *detail = 0;
    if (!workspace) return BSA_ERR_NULL_POINTER;
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    uint32_t words[2] = {0, 0};             // status code, detail (the offending block rank of a BAD_SHAPE report)
    if (cudaMemcpyAsync(words, workspace, sizeof(words), cudaMemcpyDeviceToHost, s) != cudaSuccess) return BSA_ERR_LAUNCH;
    if (cudaStreamSynchronize(s) != cudaSuccess) return BSA_ERR_LAUNCH;
    if (words[0] == 0) return BSA_OK;
    if (detail) *detail = (int32_t)words[1];
    if (cudaMemsetAsync(workspace, 0, sizeof(words), s) != cudaSuccess) return BSA_ERR_LAUNCH;
    if (cudaStreamSynchronize(s) != cudaSuccess) return BSA_ERR_LAUNCH;
    return words[0] == (uint32_t)BSA_ERR_BAD_SHAPE ? BSA_ERR_BAD_SHAPE : BSA_ERR_DEVICE_TIMEOUT;
}

extern "C" int bsa_workspace_status(void* workspace, void* stream) {
    return bsa_workspace_status_detail(workspace, stream, nullptr);
}

// ---------------------------------------------------------------------------
// bsa_matmul_noalloc: the matmul for callers that must not allocate.
//
// The matmul kernels need BSA_WORKSPACE_BYTES of device scratch (the word in which a
// kernel reports a bounded wait that ran out, plus diagnostics).  bsa_matmul takes that scratch
// from the caller.  Code that runs where cudaMalloc is off limits -- inside another
// framework's memory pool, in a real-time loop, in a plugin that was handed fixed buffers --
// has nowhere to get it from, so this entry point keeps the scratch in device memory that is
// part of the library image itself.
namespace {
constexpr size_t kStaticWorkspaceBytes = 256;      // the stated maximum of scratch this entry point can serve
constexpr int kMaxDevices = 64;
static __device__ __align__(256) unsigned char g_static_workspace[kStaticWorkspaceBytes];
}  // namespace

namespace {
// Device address of the static array on the CURRENT device (looked up once per device, no allocation).
// In host code `g_static_workspace` is only a handle of the symbol, not an address the GPU can use, and
// the address differs per device.
int static_workspace(void** out) {
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess) { cudaGetLastError(); return BSA_ERR_LAUNCH; }
    if (dev < 0 || dev >= kMaxDevices) return BSA_ERR_TOO_LARGE;
    static std::mutex mutex;
    static void* device_ptr[kMaxDevices] = {};
    std::lock_guard<std::mutex> lock(mutex);
    if (device_ptr[dev] == nullptr) {
        void* ptr = nullptr;
        if (cudaGetSymbolAddress(&ptr, g_static_workspace) != cudaSuccess || ptr == nullptr) {
            cudaGetLastError();
            return BSA_ERR_LAUNCH;
        }
        device_ptr[dev] = ptr;
    }
    *out = device_ptr[dev];
    return BSA_OK;
}
}  // namespace

extern "C" int bsa_matmul_noalloc(int mode, int dtype, int trans_a, int trans_b,
                                  const void* a, const void* b, void* c,
                                  const int32_t* blocks, const int32_t* table,
                                  int64_t nnz, int64_t groups, int64_t batches,
                                  int64_t size_m, int64_t size_n, int64_t size_k, int block,
                                  int engine, int wait_and_check, void* stream) {
    // Scratch the kernels need versus what the static array holds.
    if (BSA_WORKSPACE_BYTES > kStaticWorkspaceBytes) return BSA_ERR_WORKSPACE;
    const int checked = check_matmul_args(mode, dtype, a, b, c, blocks, table, nnz, groups, batches,
                                          size_m, size_n, size_k, block, engine);
    if (checked != BSA_OK) return checked;      // refused before the device is touched
    void* ws = nullptr;
    const int found = static_workspace(&ws);
    if (found != BSA_OK) return found;
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    // The array keeps whatever the previous call left in it; the status words must start at zero.
    if (cudaMemsetAsync(ws, 0, kStaticWorkspaceBytes, s) != cudaSuccess) { cudaGetLastError(); return BSA_ERR_LAUNCH; }
    const int st = bsa_matmul(mode, dtype, trans_a, trans_b, a, b, c, blocks, table, nnz, groups, batches,
                              size_m, size_n, size_k, block, ws, kStaticWorkspaceBytes, engine, stream);
    if (st != BSA_OK || !wait_and_check) return st;
    return bsa_workspace_status(ws, stream);
}

extern "C" int bsa_matmul_noalloc_status(void* stream) {
    void* ws = nullptr;
    const int found = static_workspace(&ws);
    if (found != BSA_OK) return found;
    return bsa_workspace_status(ws, stream);
}
