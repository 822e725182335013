// Host-side native runtime (no CUDA): asynchronous checkpoint file writer, sample-index and blend-index
// builders for the packed-document dataset, and a span gatherer over memory-mapped token files.
// Exposed to Python as the module `_mt_io`.  The logic lives in io_core.h (no torch dependency, also built as a
// sanitizer self-test); this file converts tensors to pointers and back.
#include <torch/extension.h>

#include "io_core.h"

namespace {

class AsyncFileWriter {
 public:
  explicit AsyncFileWriter(int num_threads) : core_(num_threads) {}
  void submit(const std::string& path, torch::Tensor host) {
    TORCH_CHECK(!host.is_cuda(), "submit expects a host tensor");
    TORCH_CHECK(host.is_contiguous(), "submit expects a contiguous tensor");
    auto keep = std::make_shared<torch::Tensor>(std::move(host));  // the job keeps the tensor alive
    core_.submit(path, keep->data_ptr(), static_cast<size_t>(keep->nbytes()), keep);
  }
  void wait() { core_.wait(); }
  int64_t pending() { return core_.pending(); }

 private:
  mtio::AsyncFileWriter core_;
};

// Returns [num_samples + 1, 2] int64 (see mtio::build_sample_index).
torch::Tensor build_sample_index(const torch::Tensor& doc_lengths, const torch::Tensor& document_index,
                                 int64_t seq_len, bool add_extra_token) {
  auto lens = doc_lengths.to(torch::kInt64).contiguous();
  auto order = document_index.to(torch::kInt64).contiguous();
  const auto rows = mtio::build_sample_index(lens.data_ptr<int64_t>(), order.data_ptr<int64_t>(), order.numel(),
                                             seq_len + (add_extra_token ? 1 : 0));
  auto out = torch::empty({static_cast<int64_t>(rows.size() / 2), 2}, torch::kInt64);
  std::memcpy(out.data_ptr<int64_t>(), rows.data(), rows.size() * sizeof(int64_t));
  return out;
}

// Returns (dataset_index [size] int32, dataset_sample_index [size] int64).
std::pair<torch::Tensor, torch::Tensor> build_blend_index(const torch::Tensor& weights, const torch::Tensor& lengths,
                                                          int64_t size) {
  auto w = weights.to(torch::kFloat64).contiguous();
  auto len = lengths.to(torch::kInt64).contiguous();
  TORCH_CHECK(len.numel() == w.numel(), "weights and lengths must have the same size");
  auto ds = torch::empty({size}, torch::kInt32);
  auto si = torch::empty({size}, torch::kInt64);
  mtio::build_blend_index(w.data_ptr<double>(), len.data_ptr<int64_t>(), w.numel(), size, ds.data_ptr<int32_t>(),
                          si.data_ptr<int64_t>());
  return {ds, si};
}

class MMapTokens {
 public:
  MMapTokens(const std::vector<std::string>& paths, int64_t dtype_bytes) : core_(paths, dtype_bytes) {}
  torch::Tensor gather(const torch::Tensor& byte_offsets, const torch::Tensor& counts, int64_t out_len) {
    auto off = byte_offsets.to(torch::kInt64).contiguous();
    auto cnt = counts.to(torch::kInt64).contiguous();
    TORCH_CHECK(off.numel() == cnt.numel(), "offsets and counts must have the same size");
    auto out = torch::empty({out_len}, torch::kInt32);
    core_.gather(off.data_ptr<int64_t>(), cnt.data_ptr<int64_t>(), off.numel(), out.data_ptr<int32_t>(), out_len);
    return out;
  }
  int64_t total_bytes() const { return core_.total_bytes(); }

 private:
  mtio::MMapTokens core_;
};

}  // namespace

PYBIND11_MODULE(TORCH_EXTENSION_NAME, m) {
  py::class_<AsyncFileWriter>(m, "AsyncFileWriter")
      .def(py::init<int>(), py::arg("num_threads") = 4)
      .def("submit", &AsyncFileWriter::submit, py::call_guard<py::gil_scoped_release>())
      .def("wait", &AsyncFileWriter::wait, py::call_guard<py::gil_scoped_release>())
      .def("pending", &AsyncFileWriter::pending);
  py::class_<MMapTokens>(m, "MMapTokens")
      .def(py::init<const std::vector<std::string>&, int64_t>())
      .def("gather", &MMapTokens::gather)
      .def("total_bytes", &MMapTokens::total_bytes);
  m.def("build_sample_index", &build_sample_index);
  m.def("build_blend_index", &build_blend_index);
}
