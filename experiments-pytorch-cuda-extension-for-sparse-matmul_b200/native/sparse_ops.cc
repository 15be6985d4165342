// Torch-extension binding `sparse_ops`: a thin shim from torch tensors to the
// C ABI declared in include/bsa.h.
//
// It keeps the entry point of the reference binding
// (sparse/native/sparse_kernels.cc:7-11,53-57; legacy native/sparse_ops.cc:6-10)
//     sparse_matmul(a, b, mode, row_layout, col_layout, tr_a, tr_b) -> Tensor
// with the same layout choice, shape inference and batch flattening
// (sparse_kernels.cc:12-37), and adds what the reference never bound:
// the softmax pair whose C++ signatures exist only in sparse_softmax.cu:208-236,
// a device-side layout builder and the block gather / scatter converters.
// Unlike the reference (no checks at all, uninitialised output for an unknown
// dtype or mode) every call validates its arguments and turns a non-zero
// library status into a Python exception.
#include <torch/extension.h>

#include <ATen/cuda/CUDAContext.h>
#include <c10/cuda/CUDAGuard.h>

#include <map>
#include <mutex>
#include <string>
#include <tuple>
#include <vector>

#include "bsa.h"

namespace {

using layout_tensors = std::tuple<torch::Tensor, torch::Tensor>;

void check_status(int status, const char* what) {
    TORCH_CHECK(status == BSA_OK, what, ": ", bsa_status_string(status), " (status ", status, ")");
}

int dtype_code(const torch::Tensor& t) {
    switch (t.scalar_type()) {
        case at::kFloat: return BSA_DTYPE_F32;
        case at::kHalf: return BSA_DTYPE_F16;
        case at::kBFloat16: return BSA_DTYPE_BF16;
        default: TORCH_CHECK(false, "sparse_ops: unsupported dtype ", t.scalar_type(),
                             " (float32, float16 and bfloat16 are supported)");
    }
    return -1;
}

void check_layout(const layout_tensors& layout, const torch::Device& device, const char* name) {
    const auto& blocks = std::get<0>(layout);
    const auto& table = std::get<1>(layout);
    TORCH_CHECK(blocks.scalar_type() == at::kInt && table.scalar_type() == at::kInt, name, " must hold int32 tensors");
    TORCH_CHECK(blocks.device() == device && table.device() == device, name, " must live on the operands' device");
    TORCH_CHECK(blocks.is_contiguous() && table.is_contiguous(), name, " must be contiguous");
    TORCH_CHECK(blocks.dim() == 1 && blocks.size(0) % 2 == 0 && table.dim() == 1 && table.size(0) >= 2,
                name, " has the wrong shape");
}

// One zeroed workspace per device, created on first use and kept for the
// life of the process (BSA_WORKSPACE_BYTES each).
torch::Tensor workspace_for(const torch::Device& device) {
    static std::mutex mutex;
    static std::map<int, torch::Tensor> cache;
    std::lock_guard<std::mutex> lock(mutex);
    auto it = cache.find(device.index());
    if (it == cache.end()) {
        auto ws = torch::zeros({BSA_WORKSPACE_BYTES}, torch::TensorOptions().dtype(torch::kUInt8).device(device));
        it = cache.emplace(device.index(), ws).first;
    }
    return it->second;
}

int engine_code(const std::string& engine) {
    if (engine == "auto") return BSA_ENGINE_AUTO;
    if (engine == "simt") return BSA_ENGINE_SIMT;
    if (engine == "tcgen05") return BSA_ENGINE_TCGEN05;
    TORCH_CHECK(false, "engine must be 'auto', 'simt' or 'tcgen05', got '", engine, "'");
    return -1;
}

torch::Tensor sparse_matmul(torch::Tensor a, torch::Tensor b, const std::string& mode,
                            const layout_tensors& row_layout, const layout_tensors& col_layout,
                            bool tr_a, bool tr_b, int64_t block, const std::string& engine) {
    TORCH_CHECK(mode == "sdd" || mode == "dsd" || mode == "dds",
                "mode must be 'sdd', 'dsd' or 'dds', got '", mode, "'");
    TORCH_CHECK(a.is_cuda() && b.is_cuda() && a.device() == b.device(), "a and b must be CUDA tensors on one device");
    TORCH_CHECK(a.scalar_type() == b.scalar_type(), "a and b must have the same dtype");
    const int dtype = dtype_code(a);
    check_layout(row_layout, a.device(), "row_layout");
    check_layout(col_layout, a.device(), "col_layout");
    const bool a_dense = mode[1] == 'd', b_dense = mode[2] == 'd';
    TORCH_CHECK(a.dim() >= (a_dense ? 3 : 4), "a needs at least one batch dimension");
    TORCH_CHECK(b.dim() >= (b_dense ? 3 : 4), "b needs at least one batch dimension");
    if (block == 0) block = !a_dense ? a.size(-1) : (!b_dense ? b.size(-1) : 32);
    if (!a_dense) TORCH_CHECK(a.size(-1) == block && a.size(-2) == block, "sparse a must be [..., nnz, block, block]");
    if (!b_dense) TORCH_CHECK(b.size(-1) == block && b.size(-2) == block, "sparse b must be [..., nnz, block, block]");

    // Same choice as the reference dispatcher (sparse_kernels.cc:12).
    const bool use_row = mode == "sdd" || (mode == "dsd" && !tr_a) || (mode == "dds" && tr_b);
    const auto& layout = use_row ? row_layout : col_layout;
    const auto& blocks = std::get<0>(layout);
    const auto& table = std::get<1>(layout);
    const int64_t nnz = blocks.size(0) / 2;
    const int64_t groups = table.size(0) - 1;
    const int64_t sparse_width = groups * block;

    const int64_t size_m = a_dense ? a.size(tr_a ? -1 : -2) : sparse_width;
    const int64_t size_n = b_dense ? b.size(tr_b ? -2 : -1) : sparse_width;
    const int64_t size_k = b_dense ? b.size(tr_b ? -1 : -2) : a.size(tr_a ? -2 : -1);
    if (a_dense && b_dense)
        TORCH_CHECK(a.size(tr_a ? -2 : -1) == size_k, "inner dimensions of a and b differ");
    // The extent along the axis the chosen layout does not group comes from the other layout: a dense operand
    // that is shorter than the pattern would be read beyond its end by the blocks of the last columns / rows.
    {
        const auto& other_table = std::get<1>(use_row ? col_layout : row_layout);
        const int64_t other_width = (other_table.size(0) - 1) * block;
        if (mode == "sdd") {
            TORCH_CHECK(size_n == other_width, "sdd: op(b) has ", size_n, " columns, the layout covers ", other_width);
        } else {
            TORCH_CHECK(size_k == other_width, mode, ": the dense operand's inner size is ", size_k,
                        ", the layout covers ", other_width);
        }
    }
    if (!a_dense) TORCH_CHECK(a.size(-3) == nnz, "sparse a holds ", a.size(-3), " blocks, the layout ", nnz);
    if (!b_dense) TORCH_CHECK(b.size(-3) == nnz, "sparse b holds ", b.size(-3), " blocks, the layout ", nnz);

    const auto& dense = a_dense ? a : b;
    auto shape = dense.sizes().slice(0, dense.dim() - 2).vec();
    if (mode[0] == 'd') shape.insert(shape.end(), {size_m, size_n});
    else shape.insert(shape.end(), {nnz, block, block});

    a = a.flatten(0, a_dense ? -3 : -4).contiguous();
    b = b.flatten(0, b_dense ? -3 : -4).contiguous();
    const int64_t batches = a.size(0);
    TORCH_CHECK(b.size(0) == batches, "a and b have different batch sizes (", batches, " vs ", b.size(0), ")");

    c10::cuda::CUDAGuard guard(a.device());
    torch::Tensor c = mode[0] == 'd' ? a.new_empty({batches, size_m, size_n})
                                     : a.new_empty({batches, nnz, block, block});
    if (c.numel() > 0) {
        auto ws = workspace_for(a.device());
        const int mode_code = mode == "sdd" ? BSA_MODE_SDD : (mode == "dsd" ? BSA_MODE_DSD : BSA_MODE_DDS);
        if (nnz == 0) {
            c.zero_();
        } else {
            check_status(bsa_matmul(mode_code, dtype, tr_a, tr_b, a.data_ptr(), b.data_ptr(), c.data_ptr(),
                                    blocks.data_ptr<int>(), table.data_ptr<int>(), nnz, groups, batches,
                                    size_m, size_n, size_k, static_cast<int>(block),
                                    ws.data_ptr(), BSA_WORKSPACE_BYTES, engine_code(engine),
                                    at::cuda::getCurrentCUDAStream().stream()),
                         "sparse_matmul");
        }
    }
    return c.reshape(shape);
}

torch::Tensor sparse_softmax_forward(torch::Tensor x, torch::Tensor row_blocks, torch::Tensor row_table,
                                     double scale, bool causal, c10::optional<torch::Tensor> key_padding_mask,
                                     int64_t max_row_blocks) {
    TORCH_CHECK(x.is_cuda() && x.dim() >= 4, "x must be a CUDA tensor [..., nnz, block, block]");
    check_layout({row_blocks, row_table}, x.device(), "row layout");
    const int dtype = dtype_code(x);
    const int64_t block = x.size(-1), nnz = row_blocks.size(0) / 2;
    TORCH_CHECK(x.size(-2) == block && x.size(-3) == nnz, "x must be [..., nnz, block, block] for this layout");
    const auto shape = x.sizes().vec();
    x = x.flatten(0, -4).contiguous();
    auto y = torch::empty_like(x);
    c10::cuda::CUDAGuard guard(x.device());
    const uint8_t* kpm = nullptr;
    int64_t kpm_batches = 0, kpm_stride = 0;
    torch::Tensor mask;
    if (key_padding_mask.has_value() && key_padding_mask->defined()) {
        mask = key_padding_mask->to(x.device()).ne(0).to(torch::kUInt8).contiguous();
        TORCH_CHECK(mask.dim() == 2, "key_padding_mask must be [batch, seq_k]");
        TORCH_CHECK(x.size(0) % mask.size(0) == 0, "key_padding_mask batch does not divide the flattened batch");
        kpm = mask.data_ptr<uint8_t>();
        kpm_batches = mask.size(0);
        kpm_stride = mask.size(1);
    }
    if (x.numel() > 0)
        check_status(bsa_softmax_forward(dtype, x.data_ptr(), y.data_ptr(), row_blocks.data_ptr<int>(),
                                         row_table.data_ptr<int>(), nnz, row_table.size(0) - 1, x.size(0),
                                         static_cast<int>(block), static_cast<float>(scale), causal, kpm,
                                         kpm_batches, kpm_stride, max_row_blocks,
                                         at::cuda::getCurrentCUDAStream().stream()),
                     "sparse_softmax_forward");
    return y.reshape(shape);
}

torch::Tensor sparse_softmax_backward(torch::Tensor y, torch::Tensor dy, torch::Tensor row_blocks,
                                      torch::Tensor row_table, double scale, int64_t max_row_blocks) {
    TORCH_CHECK(y.is_cuda() && dy.is_cuda() && y.dim() >= 4 && y.sizes() == dy.sizes(),
                "y and dy must be CUDA tensors of one shape [..., nnz, block, block]");
    TORCH_CHECK(y.scalar_type() == dy.scalar_type(), "y and dy must have the same dtype");
    check_layout({row_blocks, row_table}, y.device(), "row layout");
    const int dtype = dtype_code(y);
    const int64_t block = y.size(-1), nnz = row_blocks.size(0) / 2;
    TORCH_CHECK(y.size(-2) == block && y.size(-3) == nnz, "y must be [..., nnz, block, block] for this layout");
    const auto shape = y.sizes().vec();
    y = y.flatten(0, -4).contiguous();
    dy = dy.flatten(0, -4).contiguous();
    auto dx = torch::empty_like(y);
    c10::cuda::CUDAGuard guard(y.device());
    if (y.numel() > 0)
        check_status(bsa_softmax_backward(dtype, y.data_ptr(), dy.data_ptr(), dx.data_ptr(),
                                          row_blocks.data_ptr<int>(), row_table.data_ptr<int>(), nnz,
                                          row_table.size(0) - 1, y.size(0), static_cast<int>(block),
                                          static_cast<float>(scale), max_row_blocks,
                                          at::cuda::getCurrentCUDAStream().stream()),
                     "sparse_softmax_backward");
    return dx.reshape(shape);
}

// Fused block-sparse attention forward: (O, lse) = attention(Q, K, V) over the row layout.
// q [..., seq_q, d], k and v [..., seq_k, d]; 16-bit types, block 64, d = 64 or 128.
std::tuple<torch::Tensor, torch::Tensor> sparse_attention_forward(
        torch::Tensor q, torch::Tensor k, torch::Tensor v, torch::Tensor row_blocks, torch::Tensor row_table,
        int64_t block, int64_t block_cols, double scale, bool causal, c10::optional<torch::Tensor> key_padding_mask,
        bool quadrant_masks) {
    TORCH_CHECK(q.is_cuda() && k.is_cuda() && v.is_cuda(), "q, k, v must be CUDA tensors");
    TORCH_CHECK(q.dim() >= 3 && k.dim() == q.dim() && v.dim() == q.dim(), "q, k, v must be [..., seq, head_dim]");
    TORCH_CHECK(q.scalar_type() == k.scalar_type() && q.scalar_type() == v.scalar_type(), "q, k, v must share a dtype");
    check_layout({row_blocks, row_table}, q.device(), "row layout");
    const int dtype = dtype_code(q);
    const int64_t nnz = row_blocks.size(0) / 2, block_rows = row_table.size(0) - 1, d = q.size(-1);
    TORCH_CHECK(q.size(-2) == block_rows * block, "q has ", q.size(-2), " rows, the layout ", block_rows * block);
    TORCH_CHECK(k.size(-2) == block_cols * block && v.size(-2) == block_cols * block,
                "k and v must have ", block_cols * block, " rows");
    TORCH_CHECK(k.size(-1) == d && v.size(-1) == d, "q, k, v must share the head dimension");
    auto lead = q.sizes().vec();
    lead.pop_back(); lead.pop_back();
    q = q.flatten(0, -3).contiguous();
    k = k.flatten(0, -3).contiguous();
    v = v.flatten(0, -3).contiguous();
    TORCH_CHECK(k.size(0) == q.size(0) && v.size(0) == q.size(0), "q, k, v must share the leading dimensions");
    auto o = torch::empty_like(q);
    auto lse = torch::empty({q.size(0), q.size(1)}, q.options().dtype(torch::kFloat));
    c10::cuda::CUDAGuard guard(q.device());
    const uint8_t* kpm = nullptr;
    int64_t kpm_batches = 0, kpm_stride = 0;
    torch::Tensor mask;
    if (key_padding_mask.has_value() && key_padding_mask->defined()) {
        mask = key_padding_mask->to(q.device()).ne(0).to(torch::kUInt8).contiguous();
        TORCH_CHECK(mask.dim() == 2, "key_padding_mask must be [batch, seq_k]");
        TORCH_CHECK(q.size(0) % mask.size(0) == 0, "key_padding_mask batch does not divide the flattened batch");
        kpm = mask.data_ptr<uint8_t>();
        kpm_batches = mask.size(0);
        kpm_stride = mask.size(1);
    }
    if (q.numel() > 0) {
        torch::Tensor ws = workspace_for(q.device());
        check_status(bsa_attention_forward(dtype, q.data_ptr(), k.data_ptr(), v.data_ptr(), o.data_ptr(),
                                           lse.data_ptr<float>(), row_blocks.data_ptr<int>(), row_table.data_ptr<int>(),
                                           nnz, block_rows, block_cols, q.size(0), d, static_cast<int>(block),
                                           static_cast<float>(scale), causal, kpm, kpm_batches, kpm_stride, quadrant_masks,
                                           ws.data_ptr(), BSA_WORKSPACE_BYTES, at::cuda::getCurrentCUDAStream().stream()),
                     "sparse_attention_forward");
    }
    auto o_shape = lead; o_shape.push_back(q.size(1)); o_shape.push_back(d);
    auto l_shape = lead; l_shape.push_back(q.size(1));
    return {o.reshape(o_shape), lse.reshape(l_shape)};
}

// Gradients (dq, dk, dv) of sparse_attention_forward's output from the inputs, the output, its
// gradient and the log-sum-exp the forward returned (fused backward kernels: the probability
// blocks are recomputed on chip).
std::tuple<torch::Tensor, torch::Tensor, torch::Tensor> sparse_attention_backward(
        torch::Tensor q, torch::Tensor k, torch::Tensor v, torch::Tensor o, torch::Tensor dout, torch::Tensor lse,
        torch::Tensor row_blocks, torch::Tensor row_table, torch::Tensor col_blocks, torch::Tensor col_table,
        int64_t block, double scale, bool causal, c10::optional<torch::Tensor> key_padding_mask, bool quadrant_masks) {
    TORCH_CHECK(q.is_cuda() && k.is_cuda() && v.is_cuda() && o.is_cuda() && dout.is_cuda() && lse.is_cuda(),
                "all tensors must be CUDA tensors");
    TORCH_CHECK(q.dim() >= 3 && k.dim() == q.dim() && v.dim() == q.dim(), "q, k, v must be [..., seq, head_dim]");
    TORCH_CHECK(q.scalar_type() == k.scalar_type() && q.scalar_type() == v.scalar_type() &&
                q.scalar_type() == o.scalar_type() && q.scalar_type() == dout.scalar_type(), "q, k, v, o, dout must share a dtype");
    TORCH_CHECK(lse.scalar_type() == torch::kFloat, "lse must be float32");
    check_layout({row_blocks, row_table}, q.device(), "row layout");
    check_layout({col_blocks, col_table}, q.device(), "column layout");
    const int dtype = dtype_code(q);
    const int64_t nnz = row_blocks.size(0) / 2, block_rows = row_table.size(0) - 1, block_cols = col_table.size(0) - 1;
    const int64_t d = q.size(-1);
    TORCH_CHECK(col_blocks.size(0) == row_blocks.size(0), "row and column layout must describe the same blocks");
    TORCH_CHECK(q.size(-2) == block_rows * block, "q has ", q.size(-2), " rows, the layout ", block_rows * block);
    TORCH_CHECK(k.size(-2) == block_cols * block && v.size(-2) == block_cols * block,
                "k and v must have ", block_cols * block, " rows");
    TORCH_CHECK(k.size(-1) == d && v.size(-1) == d, "q, k, v must share the head dimension");
    TORCH_CHECK(o.sizes() == q.sizes() && dout.sizes() == q.sizes(), "o and dout must have q's shape");
    const auto q_shape = q.sizes().vec(), k_shape = k.sizes().vec();
    q = q.flatten(0, -3).contiguous();
    k = k.flatten(0, -3).contiguous();
    v = v.flatten(0, -3).contiguous();
    o = o.flatten(0, -3).contiguous();
    dout = dout.flatten(0, -3).contiguous();
    lse = lse.reshape({-1, q.size(1)}).contiguous();
    TORCH_CHECK(k.size(0) == q.size(0) && v.size(0) == q.size(0) && lse.size(0) == q.size(0),
                "q, k, v, lse must share the leading dimensions");
    auto dq = torch::empty_like(q), dk = torch::empty_like(k), dv = torch::empty_like(v);
    c10::cuda::CUDAGuard guard(q.device());
    const uint8_t* kpm = nullptr;
    int64_t kpm_batches = 0, kpm_stride = 0;
    torch::Tensor mask;
    if (key_padding_mask.has_value() && key_padding_mask->defined()) {
        mask = key_padding_mask->to(q.device()).ne(0).to(torch::kUInt8).contiguous();
        TORCH_CHECK(mask.dim() == 2, "key_padding_mask must be [batch, seq_k]");
        TORCH_CHECK(q.size(0) % mask.size(0) == 0, "key_padding_mask batch does not divide the flattened batch");
        kpm = mask.data_ptr<uint8_t>();
        kpm_batches = mask.size(0);
        kpm_stride = mask.size(1);
    }
    if (q.numel() > 0) {
        torch::Tensor ws = workspace_for(q.device());
        auto stats = torch::empty({q.size(0), q.size(1), 2}, q.options().dtype(torch::kFloat));
        check_status(bsa_attention_backward(dtype, q.data_ptr(), k.data_ptr(), v.data_ptr(), o.data_ptr(), dout.data_ptr(),
                                            lse.data_ptr<float>(), dq.data_ptr(), dk.data_ptr(), dv.data_ptr(),
                                            row_blocks.data_ptr<int>(), row_table.data_ptr<int>(),
                                            col_blocks.data_ptr<int>(), col_table.data_ptr<int>(),
                                            nnz, block_rows, block_cols, q.size(0), d, static_cast<int>(block),
                                            static_cast<float>(scale), causal, kpm, kpm_batches, kpm_stride, quadrant_masks,
                                            stats.data_ptr(), static_cast<size_t>(stats.numel()) * 4,
                                            ws.data_ptr(), BSA_WORKSPACE_BYTES, at::cuda::getCurrentCUDAStream().stream()),
                     "sparse_attention_backward");
    }
    return {dq.reshape(q_shape), dk.reshape(k_shape), dv.reshape(k_shape)};
}

// (row_blocks, row_table, col_blocks, col_table) of a 2-D pattern, built on
// the pattern's CUDA device.  One host read-back (the block count) sizes the
// descriptor tensors, like torch.nonzero in the reference (sparse/layout.py:8).
std::tuple<torch::Tensor, torch::Tensor, torch::Tensor, torch::Tensor> build_layout(torch::Tensor pattern) {
    TORCH_CHECK(pattern.is_cuda() && pattern.dim() == 2, "pattern must be a 2-D CUDA tensor");
    TORCH_CHECK(pattern.size(0) > 0 && pattern.size(1) > 0, "pattern must not be empty");
    int code;
    switch (pattern.scalar_type()) {
        case at::kByte: code = BSA_PATTERN_U8; break;
        case at::kBool: pattern = pattern.to(torch::kUInt8); code = BSA_PATTERN_U8; break;
        case at::kInt: code = BSA_PATTERN_I32; break;
        case at::kLong: code = BSA_PATTERN_I64; break;
        case at::kFloat: code = BSA_PATTERN_F32; break;
        default: pattern = pattern.ne(0).to(torch::kUInt8); code = BSA_PATTERN_U8; break;
    }
    pattern = pattern.contiguous();
    const int64_t rows = pattern.size(0), cols = pattern.size(1);
    c10::cuda::CUDAGuard guard(pattern.device());
    const auto opts = torch::TensorOptions().dtype(torch::kInt).device(pattern.device());
    auto row_blocks = torch::empty({2 * rows * cols}, opts), col_blocks = torch::empty({2 * rows * cols}, opts);
    auto row_table = torch::empty({rows + 1}, opts), col_table = torch::empty({cols + 1}, opts);
    auto nnz = torch::empty({1}, opts);
    check_status(bsa_layout_build(pattern.data_ptr(), code, static_cast<int>(rows), static_cast<int>(cols),
                                  row_blocks.data_ptr<int>(), row_table.data_ptr<int>(),
                                  col_blocks.data_ptr<int>(), col_table.data_ptr<int>(), nnz.data_ptr<int>(),
                                  at::cuda::getCurrentCUDAStream().stream()),
                 "build_layout");
    const int64_t n = nnz.item<int>();
    return {row_blocks.narrow(0, 0, 2 * n).clone(), row_table, col_blocks.narrow(0, 0, 2 * n).clone(), col_table};
}

torch::Tensor convert(bool to_sparse, torch::Tensor x, torch::Tensor row_blocks, int64_t rows, int64_t cols,
                      int64_t block) {
    TORCH_CHECK(x.is_cuda(), "x must be a CUDA tensor");
    check_layout({row_blocks, row_blocks.new_zeros({2})}, x.device(), "row layout");
    const int dtype = dtype_code(x);
    const int64_t nnz = row_blocks.size(0) / 2;
    c10::cuda::CUDAGuard guard(x.device());
    std::vector<int64_t> shape;
    torch::Tensor out;
    if (to_sparse) {
        TORCH_CHECK(x.dim() >= 2 && x.size(-2) == rows * block && x.size(-1) == cols * block,
                    "dense tensor must be [..., ", rows * block, ", ", cols * block, "]");
        shape = x.sizes().slice(0, x.dim() - 2).vec();
        shape.insert(shape.end(), {nnz, block, block});
        x = x.reshape({-1, rows * block, cols * block}).contiguous();
        out = x.new_empty({x.size(0), nnz, block, block});
        if (out.numel() > 0)
            check_status(bsa_dense_to_sparse(dtype, x.data_ptr(), out.data_ptr(), row_blocks.data_ptr<int>(), nnz,
                                             x.size(0), rows, cols, static_cast<int>(block),
                                             at::cuda::getCurrentCUDAStream().stream()), "to_sparse");
    } else {
        TORCH_CHECK(x.dim() >= 3 && x.size(-3) == nnz && x.size(-2) == block && x.size(-1) == block,
                    "sparse tensor must be [..., ", nnz, ", ", block, ", ", block, "]");
        shape = x.sizes().slice(0, x.dim() - 3).vec();
        shape.insert(shape.end(), {rows * block, cols * block});
        x = x.reshape({-1, nnz, block, block}).contiguous();
        out = x.new_empty({x.size(0), rows * block, cols * block});
        if (out.numel() > 0)
            check_status(bsa_sparse_to_dense(dtype, x.data_ptr(), out.data_ptr(), row_blocks.data_ptr<int>(), nnz,
                                             x.size(0), rows, cols, static_cast<int>(block),
                                             at::cuda::getCurrentCUDAStream().stream()), "to_dense");
    }
    return out.reshape(shape);
}

torch::Tensor dense_to_sparse(torch::Tensor x, torch::Tensor row_blocks, int64_t rows, int64_t cols, int64_t block) {
    return convert(true, x, row_blocks, rows, cols, block);
}
torch::Tensor sparse_to_dense(torch::Tensor x, torch::Tensor row_blocks, int64_t rows, int64_t cols, int64_t block) {
    return convert(false, x, row_blocks, rows, cols, block);
}

// The ops of this module never synchronise; a kernel that gives up on a bounded wait, or meets a
// block descriptor that does not belong to its layout, leaves a status in the module's per-device
// workspace instead.  check_device_status(device_index) synchronises the current stream of that
// device, raises RuntimeError with the status string if any kernel launched through this module on
// the device reported one since the last check, and clears the word.  Call it where results are
// consumed.
void check_device_status(int64_t device_index) {
    const torch::Device device(torch::kCUDA, static_cast<c10::DeviceIndex>(device_index));
    c10::cuda::CUDAGuard guard(device);
    auto ws = workspace_for(device);
    check_status(bsa_workspace_status(ws.data_ptr(), at::cuda::getCurrentCUDAStream().stream()),
                 "check_device_status");
}

}  // namespace

PYBIND11_MODULE(TORCH_EXTENSION_NAME, m) {
    m.def("sparse_matmul", &sparse_matmul, "Block-sparse matrix multiplication (sdd / dsd / dds).",
          py::arg("a"), py::arg("b"), py::arg("mode"), py::arg("row_layout"), py::arg("col_layout"),
          py::arg("tr_a") = false, py::arg("tr_b") = false, py::arg("block") = 0, py::arg("engine") = "auto");
    m.def("sparse_softmax_forward", &sparse_softmax_forward, "Block-sparse row softmax.",
          py::arg("x"), py::arg("row_blocks"), py::arg("row_table"), py::arg("scale") = 1.0,
          py::arg("causal") = false, py::arg("key_padding_mask") = py::none(), py::arg("max_row_blocks") = 0);
    m.def("sparse_softmax_backward", &sparse_softmax_backward, "Gradient of the block-sparse row softmax.",
          py::arg("y"), py::arg("dy"), py::arg("row_blocks"), py::arg("row_table"), py::arg("scale") = 1.0,
          py::arg("max_row_blocks") = 0);
    m.def("sparse_attention_forward", &sparse_attention_forward,
          "Fused block-sparse attention forward; returns (output, log-sum-exp).",
          py::arg("q"), py::arg("k"), py::arg("v"), py::arg("row_blocks"), py::arg("row_table"), py::arg("block"),
          py::arg("block_cols"), py::arg("scale") = 1.0, py::arg("causal") = false,
          py::arg("key_padding_mask") = py::none(), py::arg("quadrant_masks") = false);
    m.def("sparse_attention_backward", &sparse_attention_backward,
          "Fused block-sparse attention backward; returns (dq, dk, dv).",
          py::arg("q"), py::arg("k"), py::arg("v"), py::arg("o"), py::arg("dout"), py::arg("lse"),
          py::arg("row_blocks"), py::arg("row_table"), py::arg("col_blocks"), py::arg("col_table"), py::arg("block"),
          py::arg("scale") = 1.0, py::arg("causal") = false, py::arg("key_padding_mask") = py::none(),
          py::arg("quadrant_masks") = false);
    m.def("build_layout", &build_layout, "Build row / column layout metadata on the device.", py::arg("pattern"));
    m.def("dense_to_sparse", &dense_to_sparse, "Gather the layout's blocks from a dense matrix.");
    m.def("sparse_to_dense", &sparse_to_dense, "Scatter blocks into a zero-filled dense matrix.");
    m.def("check_device_status", &check_device_status, "Synchronise the device's current stream; raise if a kernel reported a time-out or a bad block descriptor since the last check.",
          py::arg("device_index") = 0);
    m.def("version", []() { return bsa_version(); });
    m.attr("WORKSPACE_BYTES") = BSA_WORKSPACE_BYTES;
}
