/*
 * bsa.h -- C ABI of the B200 (sm_100a) block-sparse attention kernel library.
 *
 * This is the drop-in boundary for the block-sparse matmul / softmax / layout
 * path of the reference torch extension.  Every entry point takes plain device
 * pointers and sizes, launches asynchronously on the stream it is given and
 * returns an `int` status (BSA_OK == 0).  No C++ exception crosses this
 * boundary and the library never allocates or frees memory on behalf of the
 * caller: outputs and the small workspace are passed in.
 *
 * Wire formats (identical to the reference, sparse/layout.py:14-38):
 *   blocks : int32[2 * nnz], interleaved (idx, packed_pos) pairs where idx is
 *            the rank of the block in row-major nonzero order (the position
 *            of its tile in the [batch, nnz, block, block] sparse storage) and
 *            packed_pos = (block_row << 16) + block_col.
 *   table  : int32[groups + 1], offset of the first block of every group
 *            (groups = block rows for the row layout, block columns for the
 *            column layout); table[groups] == nnz.
 *   The row layout lists blocks in (row, col) order, the column layout in
 *   (col, row) order.
 *
 * Reference interfaces replaced by each entry point are cited as
 * file:line relative to the reference project root.
 */
#ifndef BSA_H_
#define BSA_H_

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

/* ---- status codes ------------------------------------------------------- */
enum {
    BSA_OK = 0,
    BSA_ERR_NULL_POINTER = 1,   /* a required pointer is NULL                 */
    BSA_ERR_BAD_MODE = 2,       /* mode is not sdd / dsd / dds                */
    BSA_ERR_BAD_DTYPE = 3,      /* dtype code unknown or unsupported here     */
    BSA_ERR_BAD_SHAPE = 4,      /* a size is negative, zero where it must not
                                   be, or not a multiple of the block size    */
    BSA_ERR_BAD_BLOCK = 5,      /* block size is not 16, 32, 64 or 128        */
    BSA_ERR_ALIGNMENT = 6,      /* a pointer is not 16-byte aligned           */
    BSA_ERR_WORKSPACE = 7,      /* workspace missing or too small             */
    BSA_ERR_LAUNCH = 8,         /* the CUDA runtime refused the launch        */
    BSA_ERR_DEVICE_TIMEOUT = 9, /* a bounded wait inside a kernel ran out; the
                                   output of that launch is invalid           */
    BSA_ERR_TOO_LARGE = 10,     /* a size exceeds what the entry point handles*/
    BSA_ERR_DRIVER = 11         /* a driver entry point could not be resolved */
};

/* ---- enumerations ------------------------------------------------------- */
enum { BSA_MODE_SDD = 0, BSA_MODE_DSD = 1, BSA_MODE_DDS = 2 };
enum { BSA_DTYPE_F32 = 0, BSA_DTYPE_F16 = 1, BSA_DTYPE_BF16 = 2 };
/* element type of the 0/1 pattern given to bsa_layout_build */
enum { BSA_PATTERN_U8 = 0, BSA_PATTERN_I32 = 1, BSA_PATTERN_I64 = 2, BSA_PATTERN_F32 = 3 };
/* which kernel family bsa_matmul uses */
enum { BSA_ENGINE_AUTO = 0, BSA_ENGINE_SIMT = 1, BSA_ENGINE_TCGEN05 = 2 };

/* bytes of device workspace every matmul call needs (zero it once after
 * allocation; the library keeps it zero between successful calls) */
#define BSA_WORKSPACE_BYTES 256

/* Library version, major * 10000 + minor * 100 + patch. */
int bsa_version(void);

/* Static, human readable text for a status code. */
const char* bsa_status_string(int status);

/*
 * Build both layouts of a block pattern on the device.
 * Replaces SparseLayout.__init__ / _create_layout (sparse/layout.py:6-38),
 * which runs torch ops on the host and then copies four tensors to the GPU.
 *
 *   pattern       device pointer, rows * cols elements of pattern_dtype, row
 *                 major; any nonzero value marks a block as present
 *   row_blocks,
 *   col_blocks    device, capacity 2 * rows * cols int32 each (only the first
 *                 2 * nnz are written)
 *   row_table     device, rows + 1 int32
 *   col_table     device, cols + 1 int32
 *   nnz_out       device, one int32: number of nonzero blocks
 * rows, cols <= 65535 (the packed position holds 16 bits each).
 */
int bsa_layout_build(const void* pattern, int pattern_dtype, int rows, int cols,
                     int32_t* row_blocks, int32_t* row_table,
                     int32_t* col_blocks, int32_t* col_table,
                     int32_t* nnz_out, void* stream);

/*
 * Block-sparse matrix product C = op(A) * op(B) where exactly one of
 * C (sdd), A (dsd) or B (dds) is block-sparse.
 * Replaces sparse_matmul (sparse/native/sparse_kernels.cc:7-50) together with
 * sparse_smm_32x32x32_kernel_wrapper (sparse/native/sparse_smm_gpu.cu:270-293)
 * and sparse_hmm_32x32x32_kernel_wrapper (sparse/native/sparse_hmm_gpu.cu:320-343).
 *
 *   mode            BSA_MODE_*
 *   dtype           BSA_DTYPE_* of a, b and c (accumulation is always fp32;
 *                   fp32 inputs are multiplied in full fp32 precision or as a
 *                   3xTF32 split that keeps 1e-4 relative accuracy)
 *   trans_a/b       op() transposes the operand: the last two dims of a dense
 *                   operand are swapped in memory, a sparse operand is
 *                   transposed both in block position and inside each block
 *   a, b, c         device pointers, contiguous; dense operands are
 *                   [batches, rows, cols], sparse ones [batches, nnz, block, block]
 *   blocks, table   the layout the reference's dispatcher selects
 *                   (sparse_kernels.cc:12): the row layout for sdd, for dsd
 *                   without trans_a and for dds with trans_b; the column
 *                   layout otherwise
 *   groups          number of groups in `table` (table has groups + 1 entries)
 *   size_m/n/k      logical GEMM sizes of op(A) [m,k] * op(B) [k,n]
 *   workspace       BSA_WORKSPACE_BYTES of zeroed device memory
 *   engine          BSA_ENGINE_*; AUTO picks tcgen05 where it applies
 */
int bsa_matmul(int mode, int dtype, int trans_a, int trans_b,
               const void* a, const void* b, void* c,
               const int32_t* blocks, const int32_t* table,
               int64_t nnz, int64_t groups, int64_t batches,
               int64_t size_m, int64_t size_n, int64_t size_k, int block,
               void* workspace, size_t workspace_bytes, int engine, void* stream);

/*
 * Row softmax over the nonzero blocks of every block row:
 *   y = softmax(scale * x + mask) along each dense row, restricted to the
 *   layout; rows whose every element is masked give 0.
 * Replaces sparse_softmax_forward (sparse_softmax.cu:208-231, kernel :113-155).
 *
 *   x, y            [batches, nnz, block, block] of dtype
 *   row_blocks,
 *   row_table       the ROW layout; block_rows = groups of row_table
 *   causal          nonzero: element (q, k) with k > q (absolute positions
 *                   block_row*block+i, block_col*block+j) is masked
 *   key_padding_mask  NULL or device uint8 [kpm_batches, kpm_stride]; nonzero
 *                   marks a key position as padding (masked) for the batch
 *                   index z / (batches / kpm_batches)
 *   max_row_blocks  largest number of blocks in any block row, or 0 if not
 *                   known; a hint that lets one kernel launch cover all rows
 */
int bsa_softmax_forward(int dtype, const void* x, void* y,
                        const int32_t* row_blocks, const int32_t* row_table,
                        int64_t nnz, int64_t block_rows, int64_t batches, int block,
                        float scale, int causal,
                        const uint8_t* key_padding_mask, int64_t kpm_batches,
                        int64_t kpm_stride, int64_t max_row_blocks, void* stream);

/*
 * Gradient of bsa_softmax_forward with respect to x:
 *   dx = scale * y * (dy - sum_row(dy * y)).
 * Replaces sparse_softmax_backward (sparse_softmax.cu:233-258, kernel :165-205).
 */
int bsa_softmax_backward(int dtype, const void* y, const void* dy, void* dx,
                         const int32_t* row_blocks, const int32_t* row_table,
                         int64_t nnz, int64_t block_rows, int64_t batches, int block,
                         float scale, int64_t max_row_blocks, void* stream);

/*
 * Fused block-sparse attention forward:
 *   O = softmax_rows(scale * Q K^T + masks, restricted to the layout) V
 * in one kernel; the score / probability blocks never reach memory.
 * No single counterpart in the reference: it composes the same result from
 * sparse_matmul("sdd", tr_b) (sparse/native/sparse_kernels.cc:7-50), the
 * softmax kernels (sparse_softmax.cu:208-231) and sparse_matmul("dsd"), with
 * the [batches, nnz, block, block] tensor written and re-read in between.
 * This entry point exists beside the three unfused operators; results agree
 * with their composition within the 16-bit tolerance.
 *
 *   q               [batches, block_rows * block, head_dim]
 *   k, v            [batches, block_cols * block, head_dim]
 *   o               [batches, block_rows * block, head_dim], same dtype
 *   lse             NULL or float [batches, block_rows * block]: natural log of
 *                   the row sums of exp(scale * s + mask); -inf for rows with
 *                   no unmasked element (their output rows are 0)
 *   row_blocks,
 *   row_table       the ROW layout
 *   causal, key_padding_mask, kpm_batches, kpm_stride
 *                   as in bsa_softmax_forward
 *   quadrant_masks  0, or 1: the idx field of every descriptor holds, instead of
 *                   the block's rank, a 4-bit mask of the 32 x 32 quadrants
 *                   of the block that belong to the layout (bit 2 * row_half
 *                   + col_half); scores in the other quadrants are masked.
 *                   This is how a layout of 32 x 32 blocks runs through the
 *                   kernel: as the layout of the 64 x 64 blocks that contain
 *                   them (the kernel never uses the rank).
 * Supported: BSA_DTYPE_F16 / BSA_DTYPE_BF16, block 64, head_dim 64 or 128;
 * anything else returns BSA_ERR_BAD_DTYPE / BSA_ERR_BAD_SHAPE without
 * launching (callers then compose the unfused operators).
 */
int bsa_attention_forward(int dtype, const void* q, const void* k, const void* v, void* o, float* lse,
                          const int32_t* row_blocks, const int32_t* row_table,
                          int64_t nnz, int64_t block_rows, int64_t block_cols, int64_t batches,
                          int64_t head_dim, int block, float scale, int causal,
                          const uint8_t* key_padding_mask, int64_t kpm_batches, int64_t kpm_stride,
                          int quadrant_masks,
                          void* workspace, size_t workspace_bytes, void* stream);

/*
 * Fused block-sparse attention backward: dQ, dK, dV of bsa_attention_forward's
 * output from q, k, v, o, the output gradient `dout` and the forward's `lse`;
 * the probability and score-gradient blocks never reach memory.  The
 * reference composes the same gradients from its matmul in sdd / dsd mode
 * (sparse/matmul.py:30-50 over sparse/native/sparse_kernels.cc:7-50) and its
 * softmax backward (sparse_softmax.cu:233-258).  Two launches at head dim 64:
 * dQ by block rows (ROW layout; it also computes the per-row statistics and
 * leaves them in `stats`), dK and dV by block columns (COLUMN layout); at
 * head dim 128 a launch of its own computes the statistics first.
 *
 *   q, o, dout, dq  [batches, block_rows * block, head_dim]
 *   k, v, dk, dv    [batches, block_cols * block, head_dim]
 *   lse             float [batches, block_rows * block] as written by the forward
 *   stats           scratch of at least batches * block_rows * block * 8 bytes,
 *                   16-byte aligned (`stats_bytes` = its size)
 *   masks, scale, quadrant_masks
 *                   as given to the forward (with quadrant masks in both layouts)
 * Supported combinations and error codes as for bsa_attention_forward.
 */
int bsa_attention_backward(int dtype, const void* q, const void* k, const void* v, const void* o,
                           const void* dout, const float* lse, void* dq, void* dk, void* dv,
                           const int32_t* row_blocks, const int32_t* row_table,
                           const int32_t* col_blocks, const int32_t* col_table,
                           int64_t nnz, int64_t block_rows, int64_t block_cols, int64_t batches,
                           int64_t head_dim, int block, float scale, int causal,
                           const uint8_t* key_padding_mask, int64_t kpm_batches, int64_t kpm_stride,
                           int quadrant_masks,
                           void* stats, size_t stats_bytes,
                           void* workspace, size_t workspace_bytes, void* stream);

/*
 * Gather the blocks of a dense [batches, rows*block, cols*block] matrix into
 * sparse storage (to_sparse, sparse/layout.py:40-45) or scatter them back
 * with zeros elsewhere (to_dense, sparse/layout.py:47-57).  `blocks` is the
 * ROW layout.
 */
int bsa_dense_to_sparse(int dtype, const void* dense, void* sparse,
                        const int32_t* row_blocks, int64_t nnz, int64_t batches,
                        int64_t rows, int64_t cols, int block, void* stream);
int bsa_sparse_to_dense(int dtype, const void* sparse, void* dense,
                        const int32_t* row_blocks, int64_t nnz, int64_t batches,
                        int64_t rows, int64_t cols, int block, void* stream);

/*
 * Read the device status word of a workspace (synchronises `stream`).
 * Returns BSA_OK; BSA_ERR_DEVICE_TIMEOUT if a kernel that used this workspace
 * gave up on a bounded wait (its output is invalid); or BSA_ERR_BAD_SHAPE if a
 * kernel met a block descriptor that does not belong to its layout (a rank
 * outside [0, nnz): the block was skipped).  The word is cleared on return.
 * bsa_workspace_status_detail also hands back the second workspace word in
 * `*detail` (may be NULL): for BSA_ERR_BAD_SHAPE the offending rank, else 0.
 */
int bsa_workspace_status(void* workspace, void* stream);
int bsa_workspace_status_detail(void* workspace, void* stream, int32_t* detail);

/*
 * bsa_matmul for callers that cannot allocate device memory.
 * No counterpart in the reference (its binding allocates through torch on every call).
 *
 * Same product, same arguments and same kernels as bsa_matmul, except that the
 * BSA_WORKSPACE_BYTES of scratch are not passed in: they live in a fixed
 * 256-byte array in the library's own device image (one copy per GPU that
 * loads the library, held until the process exits).  This is for code that
 * runs where cudaMalloc is not an option -- a plugin inside another
 * framework's memory pool, a latency-critical loop, a host that was only
 * handed fixed buffers.  The entry point calls no cudaMalloc, cudaFree or
 * other allocating routine; inputs and the output are still the caller's.
 *
 *   wait_and_check  0: return right after the asynchronous launch.  A time-out
 *                   inside the kernels is then reported only if the caller
 *                   reads it with bsa_matmul_noalloc_status before the next
 *                   call (which clears the array); use 0 inside a stream
 *                   capture, where synchronising is not allowed.
 *                   nonzero: synchronise `stream` and return
 *                   BSA_ERR_DEVICE_TIMEOUT if a kernel gave up on a bounded wait.
 *
 * Limits.  The scratch requirement of the kernels is fixed (it does not grow
 * with the problem); should it ever exceed the 256 bytes of the static array
 * the call is refused with BSA_ERR_WORKSPACE.  At most 64 devices.
 * The array used is the one of the device that is CURRENT in the calling
 * thread (cudaGetDevice), which must be the device `stream` and the operands
 * belong to.  The first call on each device looks up the array's device
 * address; make it before any stream capture.  All calls on a device share the
 * one array and each call clears it first, so two calls whose kernels overlap
 * on the GPU (different streams or threads) race on the status words:
 * serialise them.
 *
 * bsa_matmul_noalloc_status synchronises `stream`, then returns and clears the
 * status the last bsa_matmul_noalloc call on the current device left in the
 * array (as bsa_workspace_status does for a caller's workspace).
 */
int bsa_matmul_noalloc(int mode, int dtype, int trans_a, int trans_b,
                       const void* a, const void* b, void* c,
                       const int32_t* blocks, const int32_t* table,
                       int64_t nnz, int64_t groups, int64_t batches,
                       int64_t size_m, int64_t size_n, int64_t size_k, int block,
                       int engine, int wait_and_check, void* stream);
int bsa_matmul_noalloc_status(void* stream);

#ifdef __cplusplus
}
#endif
#endif /* BSA_H_ */
