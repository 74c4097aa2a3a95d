// Torch binding `rode_sddmm_cuda`: the Python entry of the RoDe SDDMM path.
//
// Mirrors the module the reference builds from RoDe_SDDMM/rode_sddmm_cuda.cu (functions
// `preprocess` :54-131 and `sddmm_forward` :136-249, module definition :254-278): same
// function names, argument order, checks and return shapes.  It contains no kernels; it
// turns tensors into pointers and calls the C ABI of librode_b200.so.
//
// Differences from the reference binding:
//   * preprocess runs the row decomposition on the GPU.  A CPU row_offsets tensor (the
//     reference's calling convention) is copied to the current CUDA device, decomposed
//     there, and the results are returned as CPU tensors; a CUDA row_offsets tensor gives
//     CUDA results without any host round trip except the two counts.
//   * sddmm_forward launches on torch's current stream (block part) and one side stream
//     from torch's pool (residue part) joined back with an event, instead of creating,
//     synchronising and destroying two streams per call
//     (RoDe_SDDMM/rode_sddmm_cuda.cu:203-246); it does not block the host.
//   * k_version may also be 64.
//   * spmm_forward and hot_columns are new: the reference has no Python entry for SpMM.
#include <ATen/cuda/CUDAContext.h>
#include <ATen/cuda/CUDAEvent.h>
#include <c10/cuda/CUDAGuard.h>
#include <c10/cuda/CUDAStream.h>
#include <torch/extension.h>

#include <tuple>

#include "rode_b200.h"

namespace {

#define RODE_CHECK_CUDA(x) TORCH_CHECK((x).device().is_cuda(), #x " must be a CUDA tensor")
#define RODE_CHECK_CONTIGUOUS(x) TORCH_CHECK((x).is_contiguous(), #x " must be contiguous")
#define RODE_CHECK_INPUT(x) \
    RODE_CHECK_CUDA(x);     \
    RODE_CHECK_CONTIGUOUS(x)
#define RODE_CHECK_FLOAT(x) TORCH_CHECK((x).dtype() == torch::kFloat32, #x " must be float32")
#define RODE_CHECK_INT(x) TORCH_CHECK((x).dtype() == torch::kInt32, #x " must be int32")

void check_status(int status) { TORCH_CHECK(status == RODE_OK, "rode_b200: ", rode_last_error()); }

// Runs `launch(stream1, stream2)` with the block work on the current stream and the residue
// work on a pool stream forked from it and joined back into it.
template <typename F>
void fork_join(const c10::Device &device, F launch) {
    auto cur = at::cuda::getCurrentCUDAStream(device.index());
    auto side = at::cuda::getStreamFromPool(false, device.index());
    at::cuda::CUDAEvent fork, join;
    fork.record(cur);
    fork.block(side);
    launch(cur.stream(), side.stream());
    join.record(side);
    join.block(cur);
}

std::tuple<torch::Tensor, torch::Tensor, torch::Tensor, int, int> py_preprocess(torch::Tensor row_offsets, int nnz,
                                                                                 int seg_length, int k_block,
                                                                                 int vec_len) {
    TORCH_CHECK(row_offsets.dtype() == torch::kInt32, "row_offsets must be int32");
    TORCH_CHECK(row_offsets.dim() == 1 && row_offsets.size(0) >= 1, "row_offsets must have m + 1 entries");
    TORCH_CHECK(at::cuda::is_available(), "rode_b200 needs a CUDA device; there is no CPU path");
    const bool on_host = row_offsets.device().is_cpu();
    torch::Tensor rp = (on_host ? row_offsets.to(torch::kCUDA) : row_offsets).contiguous();
    const c10::cuda::CUDAGuard guard(rp.device());
    const int m = static_cast<int>(rp.size(0)) - 1;

    long long cap = 0;
    check_status(rode_preprocess_capacity(seg_length, vec_len, m, nnz, &cap));
    size_t ws_bytes = 0;
    check_status(rode_preprocess_workspace_bytes(m, &ws_bytes));
    auto opts = torch::TensorOptions().dtype(torch::kInt32).device(rp.device());
    torch::Tensor blk = torch::empty({std::max<long long>(cap, 1)}, opts);
    torch::Tensor st = torch::empty({cap + 1}, opts);
    torch::Tensor res = torch::empty({std::max(m, 1)}, opts);
    torch::Tensor counts = torch::empty({2}, opts);
    torch::Tensor ws = torch::empty({static_cast<long long>(ws_bytes)}, opts.dtype(torch::kUInt8));
    auto stream = at::cuda::getCurrentCUDAStream(rp.device().index());
    check_status(rode_preprocess(seg_length, k_block, vec_len, m, rp.data_ptr<int>(), blk.data_ptr<int>(),
                                 st.data_ptr<int>(), res.data_ptr<int>(), counts.data_ptr<int>(),
                                 counts.data_ptr<int>() + 1, ws.data_ptr(), ws_bytes, stream.stream()));
    torch::Tensor counts_host = counts.cpu();  // synchronises the stream
    const int n_blk = counts_host.data_ptr<int>()[0];
    const int n_res = counts_host.data_ptr<int>()[1];
    // Shapes as the reference returns them: [max(n_blk,1)], [n_blk + 1], [max(n_res,1)].
    blk = blk.narrow(0, 0, std::max(n_blk, 1));
    st = st.narrow(0, 0, n_blk + 1);
    res = res.narrow(0, 0, std::max(n_res, 1));
    if (on_host) return std::make_tuple(blk.cpu(), st.cpu(), res.cpu(), n_blk, n_res);
    return std::make_tuple(blk.contiguous(), st.contiguous(), res.contiguous(), n_blk, n_res);
}

torch::Tensor py_sddmm_forward(torch::Tensor block_indices, torch::Tensor residue_indices, torch::Tensor st_offsets,
                                 int m1, int m2, torch::Tensor row_offsets, torch::Tensor column_indices,
                                 torch::Tensor values, int m, int n, torch::Tensor lhs_matrix,
                                 torch::Tensor rhs_matrix, int k_version) {
    RODE_CHECK_INPUT(block_indices);
    RODE_CHECK_INPUT(residue_indices);
    RODE_CHECK_INPUT(st_offsets);
    RODE_CHECK_INPUT(row_offsets);
    RODE_CHECK_INPUT(column_indices);
    RODE_CHECK_INPUT(values);
    RODE_CHECK_INPUT(lhs_matrix);
    RODE_CHECK_INPUT(rhs_matrix);
    RODE_CHECK_INT(block_indices);
    RODE_CHECK_INT(residue_indices);
    RODE_CHECK_INT(st_offsets);
    RODE_CHECK_INT(row_offsets);
    RODE_CHECK_INT(column_indices);
    RODE_CHECK_FLOAT(values);
    RODE_CHECK_FLOAT(lhs_matrix);
    RODE_CHECK_FLOAT(rhs_matrix);

    const int k = static_cast<int>(lhs_matrix.size(1));
    TORCH_CHECK(k_version > 0 && k_version % 4 == 0 && k_version <= 256,
                "k_version must be a multiple of 4, at most 256");
    TORCH_CHECK(k == k_version, "k dimension must match k_version");
    TORCH_CHECK(lhs_matrix.size(0) == m, "lhs_matrix rows must equal m");
    TORCH_CHECK(rhs_matrix.size(0) == n, "rhs_matrix rows must equal n");
    TORCH_CHECK(rhs_matrix.size(1) == k, "rhs_matrix cols must equal k");
    TORCH_CHECK(row_offsets.size(0) == m + 1, "row_offsets must have m + 1 entries");

    const c10::cuda::CUDAGuard guard(values.device());
    torch::Tensor out = torch::zeros({values.size(0)}, values.options());
    if (m1 == 0 && m2 == 0) return out;
    fork_join(values.device(), [&](cudaStream_t s1, cudaStream_t s2) {
        check_status(rode_sddmm_f32(m1, m2, n, k, block_indices.data_ptr<int>(), residue_indices.data_ptr<int>(),
                                    st_offsets.data_ptr<int>(), row_offsets.data_ptr<int>(),
                                    column_indices.data_ptr<int>(), values.data_ptr<float>(),
                                    lhs_matrix.data_ptr<float>(), rhs_matrix.data_ptr<float>(), out.data_ptr<float>(),
                                    s1, s2));
    });
    return out;
}

// Popularity bitmap of the columns for spmm_forward's `hot_columns` argument (rode_hot_columns),
// or None when the library finds that marks would not help.  Reads the flag word back.
c10::optional<torch::Tensor> py_hot_columns(torch::Tensor column_indices, int n_cols, int64_t dense_row_bytes,
                                            int64_t budget_bytes) {
    RODE_CHECK_INPUT(column_indices);
    RODE_CHECK_INT(column_indices);
    TORCH_CHECK(n_cols >= 0 && dense_row_bytes > 0 && budget_bytes >= 0, "bad size argument");
    const c10::cuda::CUDAGuard guard(column_indices.device());
    size_t words = 0, ws_bytes = 0;
    check_status(rode_hot_columns_words(n_cols, &words));
    check_status(rode_hot_columns_workspace_bytes(n_cols, &ws_bytes));
    auto opts = column_indices.options();
    torch::Tensor bitmap = torch::empty({static_cast<long long>(words)}, opts);
    torch::Tensor ws = torch::empty({static_cast<long long>(ws_bytes)}, opts.dtype(torch::kUInt8));
    auto stream = at::cuda::getCurrentCUDAStream(column_indices.device().index());
    check_status(rode_hot_columns(column_indices.numel(), n_cols, column_indices.data_ptr<int>(),
                                  static_cast<size_t>(dense_row_bytes), static_cast<size_t>(budget_bytes),
                                  reinterpret_cast<unsigned *>(bitmap.data_ptr<int>()), ws.data_ptr(), ws_bytes,
                                  stream.stream()));
    const bool useful = bitmap[static_cast<long long>(words) - 1].item<int>() != 0;
    if (!useful) return c10::nullopt;
    return bitmap;
}

torch::Tensor py_spmm_forward(torch::Tensor block_indices, torch::Tensor residue_indices, torch::Tensor st_offsets,
                                int m1, int m2, torch::Tensor row_offsets, torch::Tensor column_indices,
                                torch::Tensor values, int m, int k, torch::Tensor dense,
                                c10::optional<torch::Tensor> hot_columns) {
    RODE_CHECK_INPUT(block_indices);
    RODE_CHECK_INPUT(residue_indices);
    RODE_CHECK_INPUT(st_offsets);
    RODE_CHECK_INPUT(row_offsets);
    RODE_CHECK_INPUT(column_indices);
    RODE_CHECK_INPUT(values);
    RODE_CHECK_INPUT(dense);
    RODE_CHECK_INT(block_indices);
    RODE_CHECK_INT(residue_indices);
    RODE_CHECK_INT(st_offsets);
    RODE_CHECK_INT(row_offsets);
    RODE_CHECK_INT(column_indices);
    TORCH_CHECK(values.dtype() == torch::kFloat32 || values.dtype() == torch::kFloat64,
                "values must be float32 or float64");
    TORCH_CHECK(dense.dtype() == values.dtype(), "dense must have the dtype of values");
    TORCH_CHECK(dense.dim() == 2 && dense.size(0) == k, "dense must be [k, n]");
    TORCH_CHECK(row_offsets.size(0) == m + 1, "row_offsets must have m + 1 entries");
    const int n = static_cast<int>(dense.size(1));

    const c10::cuda::CUDAGuard guard(values.device());
    torch::Tensor out = torch::zeros({m, n}, dense.options());
    if (m1 == 0 && m2 == 0) return out;
    size_t ws_bytes = 0;
    check_status(rode_spmm_workspace_bytes(m1, n, static_cast<int>(dense.element_size()), &ws_bytes));
    torch::Tensor ws = torch::empty({static_cast<long long>(std::max<size_t>(ws_bytes, 16))},
                                    dense.options().dtype(torch::kUInt8));
    const unsigned *hot = nullptr;
    if (hot_columns.has_value()) {
        RODE_CHECK_INPUT(*hot_columns);
        RODE_CHECK_INT(*hot_columns);
        TORCH_CHECK(hot_columns->numel() == (static_cast<long long>(k) + 31) / 32 + 1,
                    "hot_columns must come from hot_columns() for this matrix");
        hot = reinterpret_cast<const unsigned *>(hot_columns->data_ptr<int>());
    }
    fork_join(values.device(), [&](cudaStream_t s1, cudaStream_t s2) {
        if (dense.dtype() == torch::kFloat32)
            check_status(rode_spmm_f32_hot(m1, m2, k, n, values.data_ptr<float>(), column_indices.data_ptr<int>(),
                                           row_offsets.data_ptr<int>(), block_indices.data_ptr<int>(),
                                           residue_indices.data_ptr<int>(), st_offsets.data_ptr<int>(),
                                           dense.data_ptr<float>(), out.data_ptr<float>(), ws.data_ptr(), ws_bytes,
                                           hot, s1, s2));
        else
            check_status(rode_spmm_f64_hot(m1, m2, k, n, values.data_ptr<double>(), column_indices.data_ptr<int>(),
                                           row_offsets.data_ptr<int>(), block_indices.data_ptr<int>(),
                                           residue_indices.data_ptr<int>(), st_offsets.data_ptr<int>(),
                                           dense.data_ptr<double>(), out.data_ptr<double>(), ws.data_ptr(), ws_bytes,
                                           hot, s1, s2));
    });
    // The workspace is used by the block and fix-up kernels on the current stream and, for its
    // claim counters, by the residue kernel on the side stream; the side stream was joined back
    // into the current one, so the caching allocator may reuse the buffer after this call.
    return out;
}

}  // namespace

PYBIND11_MODULE(TORCH_EXTENSION_NAME, m) {
    m.def("preprocess", &py_preprocess, "RoDe CSR row decomposition (GPU)", py::arg("row_offsets"), py::arg("nnz"),
          py::arg("seg_length"), py::arg("k_block"), py::arg("vec_len"));
    m.def("sddmm_forward", &py_sddmm_forward, "RoDe SDDMM forward (CUDA)", py::arg("block_indices"),
          py::arg("residue_indices"), py::arg("st_offsets"), py::arg("m1"), py::arg("m2"), py::arg("row_offsets"),
          py::arg("column_indices"), py::arg("values"), py::arg("m"), py::arg("n"), py::arg("lhs_matrix"),
          py::arg("rhs_matrix"), py::arg("k_version"));
    m.def("spmm_forward", &py_spmm_forward, "RoDe SpMM forward (CUDA)", py::arg("block_indices"),
          py::arg("residue_indices"), py::arg("st_offsets"), py::arg("m1"), py::arg("m2"), py::arg("row_offsets"),
          py::arg("column_indices"), py::arg("values"), py::arg("m"), py::arg("k"), py::arg("dense"),
          py::arg("hot_columns") = py::none());
    m.def("hot_columns", &py_hot_columns, "Column popularity bitmap for spmm_forward, or None (CUDA)",
          py::arg("column_indices"), py::arg("n_cols"), py::arg("dense_row_bytes"), py::arg("budget_bytes") = 0);
}
