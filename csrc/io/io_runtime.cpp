// Host-side native runtime (no CUDA): asynchronous checkpoint file writer, sample-index and blend-index
// builders for the packed-document dataset, and a span gatherer over memory-mapped token files.
// Exposed to Python as the module `_mt_io`.
#include <torch/extension.h>

#include <fcntl.h>
#include <sys/mman.h>
#include <sys/stat.h>
#include <unistd.h>

#include <atomic>
#include <condition_variable>
#include <cstring>
#include <deque>
#include <mutex>
#include <stdexcept>
#include <string>
#include <thread>
#include <vector>

namespace {

// ------------------------------------------------------------------------------------ async file writer
// Jobs are (path, host tensor) pairs; worker threads write each buffer with pwrite, fsync, and rename the
// temporary file into place, so a reader never sees a half-written file.  The tensor is kept alive by the job.
class AsyncFileWriter {
 public:
  explicit AsyncFileWriter(int num_threads) {
    if (num_threads < 1) num_threads = 1;
    for (int i = 0; i < num_threads; ++i) workers_.emplace_back([this] { run(); });
  }
  ~AsyncFileWriter() {
    {
      std::lock_guard<std::mutex> lk(mu_);
      stop_ = true;
    }
    cv_.notify_all();
    for (auto& t : workers_) t.join();
  }
  void submit(const std::string& path, torch::Tensor host) {
    TORCH_CHECK(!host.is_cuda(), "submit expects a host tensor");
    TORCH_CHECK(host.is_contiguous(), "submit expects a contiguous tensor");
    {
      std::lock_guard<std::mutex> lk(mu_);
      jobs_.push_back({path, std::move(host)});
      ++pending_;
    }
    cv_.notify_one();
  }
  // Blocks until every submitted job has been written; rethrows the first I/O error.
  void wait() {
    std::unique_lock<std::mutex> lk(mu_);
    done_cv_.wait(lk, [this] { return pending_ == 0; });
    if (!error_.empty()) {
      std::string e = error_;
      error_.clear();
      throw std::runtime_error(e);
    }
  }
  int64_t pending() {
    std::lock_guard<std::mutex> lk(mu_);
    return pending_;
  }

 private:
  struct Job {
    std::string path;
    torch::Tensor data;
  };
  void run() {
    for (;;) {
      Job job;
      {
        std::unique_lock<std::mutex> lk(mu_);
        cv_.wait(lk, [this] { return stop_ || !jobs_.empty(); });
        if (jobs_.empty()) return;
        job = std::move(jobs_.front());
        jobs_.pop_front();
      }
      std::string err = write_one(job);
      {
        std::lock_guard<std::mutex> lk(mu_);
        if (!err.empty() && error_.empty()) error_ = err;
        --pending_;
      }
      done_cv_.notify_all();
    }
  }
  static std::string write_one(const Job& job) {
    const std::string tmp = job.path + ".tmp";
    int fd = ::open(tmp.c_str(), O_WRONLY | O_CREAT | O_TRUNC, 0644);
    if (fd < 0) return "cannot open " + tmp + ": " + std::strerror(errno);
    const char* p = static_cast<const char*>(job.data.data_ptr());
    size_t left = static_cast<size_t>(job.data.nbytes());
    off_t off = 0;
    while (left > 0) {
      ssize_t n = ::pwrite(fd, p + off, left > (1u << 30) ? (1u << 30) : left, off);
      if (n < 0) {
        std::string e = "write failed for " + tmp + ": " + std::strerror(errno);
        ::close(fd);
        return e;
      }
      off += n;
      left -= static_cast<size_t>(n);
    }
    ::fsync(fd);
    ::close(fd);
    if (::rename(tmp.c_str(), job.path.c_str()) != 0) return "rename failed for " + job.path;
    return "";
  }
  std::mutex mu_;
  std::condition_variable cv_, done_cv_;
  std::deque<Job> jobs_;
  std::vector<std::thread> workers_;
  int64_t pending_ = 0;
  bool stop_ = false;
  std::string error_;
};

// ------------------------------------------------------------------------------------ sample index
// Documents (in the order given by document_index) are laid end to end and cut into consecutive samples of
// `seq_len + add_extra_token` tokens.  Row i of the result is (position in document_index, offset inside that
// document) where sample i starts; row i+1 is where it ends.  A boundary that falls exactly on a document end
// is recorded as (doc, doc_len).  Returns [num_samples + 1, 2] int64.
torch::Tensor build_sample_index(const torch::Tensor& doc_lengths, const torch::Tensor& document_index,
                                 int64_t seq_len, bool add_extra_token) {
  auto lens = doc_lengths.to(torch::kInt64).contiguous();
  auto order = document_index.to(torch::kInt64).contiguous();
  const int64_t* L = lens.data_ptr<int64_t>();
  const int64_t* O = order.data_ptr<int64_t>();
  const int64_t n_docs = order.numel();
  const int64_t target = seq_len + (add_extra_token ? 1 : 0);
  std::vector<int64_t> rows = {0, 0};
  int64_t doc_pos = 0, offset = 0, remaining = target;
  while (doc_pos < n_docs) {
    const int64_t doc_len = L[O[doc_pos]];
    const int64_t available = doc_len - offset;
    if (available <= 0) {
      ++doc_pos;
      offset = 0;
      continue;
    }
    if (available >= remaining) {
      offset += remaining;
      rows.push_back(doc_pos);
      rows.push_back(offset);
      remaining = target;
      if (offset >= doc_len) {
        ++doc_pos;
        offset = 0;
      }
    } else {
      remaining -= available;
      ++doc_pos;
      offset = 0;
    }
  }
  auto out = torch::empty({static_cast<int64_t>(rows.size() / 2), 2}, torch::kInt64);
  std::memcpy(out.data_ptr<int64_t>(), rows.data(), rows.size() * sizeof(int64_t));
  return out;
}

// Greedy weighted interleave: position i goes to the source whose realised count lags weight * (i + 1) the most
// (lowest index wins ties); the sample taken from it is that source's running counter modulo its length.
// Returns (dataset_index [size] int32, dataset_sample_index [size] int64).
std::pair<torch::Tensor, torch::Tensor> build_blend_index(const torch::Tensor& weights, const torch::Tensor& lengths,
                                                          int64_t size) {
  auto w = weights.to(torch::kFloat64).contiguous();
  auto len = lengths.to(torch::kInt64).contiguous();
  const int64_t n = w.numel();
  TORCH_CHECK(len.numel() == n, "weights and lengths must have the same size");
  const double* W = w.data_ptr<double>();
  const int64_t* Ln = len.data_ptr<int64_t>();
  double total = 0;
  for (int64_t k = 0; k < n; ++k) total += W[k];
  auto ds = torch::empty({size}, torch::kInt32);
  auto si = torch::empty({size}, torch::kInt64);
  int32_t* D = ds.data_ptr<int32_t>();
  int64_t* I = si.data_ptr<int64_t>();
  std::vector<int64_t> counts(n, 0);
  for (int64_t i = 0; i < size; ++i) {
    int64_t best = 0;
    double best_err = -1e300;
    for (int64_t k = 0; k < n; ++k) {
      const double err = (W[k] / total) * static_cast<double>(i + 1) - static_cast<double>(counts[k]);
      if (err > best_err) {
        best_err = err;
        best = k;
      }
    }
    D[i] = static_cast<int32_t>(best);
    I[i] = Ln[best] > 0 ? counts[best] % Ln[best] : 0;
    ++counts[best];
  }
  return {ds, si};
}

// ------------------------------------------------------------------------------------ mmap token reader
// Read-only mapping of one or more token files that logically form one array of `dtype_bytes`-sized tokens.
class MMapTokens {
 public:
  MMapTokens(const std::vector<std::string>& paths, int64_t dtype_bytes) : dtype_bytes_(dtype_bytes) {
    int64_t start = 0;
    for (const auto& p : paths) {
      int fd = ::open(p.c_str(), O_RDONLY);
      if (fd < 0) throw std::runtime_error("cannot open " + p);
      struct stat st;
      ::fstat(fd, &st);
      void* addr = st.st_size > 0 ? ::mmap(nullptr, st.st_size, PROT_READ, MAP_PRIVATE, fd, 0) : nullptr;
      ::close(fd);
      if (addr == MAP_FAILED) throw std::runtime_error("mmap failed for " + p);
      parts_.push_back({static_cast<const char*>(addr), static_cast<int64_t>(st.st_size), start});
      start += st.st_size;
    }
    total_bytes_ = start;
  }
  ~MMapTokens() {
    for (auto& p : parts_)
      if (p.addr) ::munmap(const_cast<char*>(p.addr), p.size);
  }
  // Copy the token spans [byte_offset[i], byte_offset[i] + count[i]*dtype_bytes) back to back into one int32 row.
  torch::Tensor gather(const torch::Tensor& byte_offsets, const torch::Tensor& counts, int64_t out_len) {
    auto off = byte_offsets.contiguous();
    auto cnt = counts.contiguous();
    auto out = torch::zeros({out_len}, torch::kInt32);
    int32_t* dst = out.data_ptr<int32_t>();
    int64_t pos = 0;
    for (int64_t i = 0; i < off.numel(); ++i) {
      const int64_t n = cnt.data_ptr<int64_t>()[i];
      int64_t b = off.data_ptr<int64_t>()[i];
      for (int64_t t = 0; t < n && pos < out_len; ++t, ++pos, b += dtype_bytes_) dst[pos] = read_token(b);
    }
    return out;
  }
  int64_t total_bytes() const { return total_bytes_; }

 private:
  struct Part {
    const char* addr;
    int64_t size;
    int64_t start;
  };
  int32_t read_token(int64_t byte) const {
    if (byte < 0 || byte + dtype_bytes_ > total_bytes_) throw std::out_of_range("token offset outside the data files");
    size_t lo = 0, hi = parts_.size();
    while (hi - lo > 1) {
      size_t mid = (lo + hi) / 2;
      if (parts_[mid].start <= byte) lo = mid;
      else hi = mid;
    }
    const char* p = parts_[lo].addr + (byte - parts_[lo].start);
    switch (dtype_bytes_) {
      case 1: return *reinterpret_cast<const uint8_t*>(p);
      case 2: { uint16_t v; std::memcpy(&v, p, 2); return v; }
      case 4: { int32_t v; std::memcpy(&v, p, 4); return v; }
      default: { int64_t v; std::memcpy(&v, p, 8); return static_cast<int32_t>(v); }
    }
  }
  std::vector<Part> parts_;
  int64_t dtype_bytes_;
  int64_t total_bytes_ = 0;
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
