// Torch-free core of the host-side I/O runtime: asynchronous file writer, sample-index and blend-index builders for
// the packed-document dataset, and a span gatherer over memory-mapped token files.  `io_runtime.cpp` wraps these for
// Python; `io_selftest.cpp` exercises them as a plain program so that they can run under the address, undefined-
// behaviour and thread sanitizers without an interpreter in the process.
#pragma once

#include <fcntl.h>
#include <sys/mman.h>
#include <sys/stat.h>
#include <unistd.h>

#include <cerrno>
#include <condition_variable>
#include <cstdint>
#include <cstring>
#include <deque>
#include <memory>
#include <mutex>
#include <stdexcept>
#include <string>
#include <thread>
#include <vector>

namespace mtio {

// ------------------------------------------------------------------------------------ async file writer
// Jobs are (path, host buffer) pairs; worker threads write each buffer with pwrite, fsync, and rename the
// temporary file into place, so a reader never sees a half-written file.  `keepalive` owns the buffer until the
// job has been written.
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
  AsyncFileWriter(const AsyncFileWriter&) = delete;
  AsyncFileWriter& operator=(const AsyncFileWriter&) = delete;

  void submit(const std::string& path, const void* data, size_t bytes, std::shared_ptr<void> keepalive) {
    {
      std::lock_guard<std::mutex> lk(mu_);
      jobs_.push_back({path, data, bytes, std::move(keepalive)});
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
    const void* data = nullptr;
    size_t bytes = 0;
    std::shared_ptr<void> keepalive;
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
      job.keepalive.reset();
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
    const char* p = static_cast<const char*>(job.data);
    size_t left = job.bytes;
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
// Documents (in the order given by `order`) are laid end to end and cut into consecutive samples of `target`
// tokens.  Row i of the result is (position in `order`, offset inside that document) where sample i starts; row
// i+1 is where it ends.  A boundary that falls exactly on a document end is recorded as (doc, doc_len).
// Returns the rows flattened: 2 * (num_samples + 1) values.
inline std::vector<int64_t> build_sample_index(const int64_t* doc_lengths, const int64_t* order, int64_t n_docs,
                                               int64_t target) {
  std::vector<int64_t> rows = {0, 0};
  if (target <= 0) return rows;
  int64_t doc_pos = 0, offset = 0, remaining = target;
  while (doc_pos < n_docs) {
    const int64_t doc_len = doc_lengths[order[doc_pos]];
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
  return rows;
}

// Greedy weighted interleave: position i goes to the source whose realised count lags weight * (i + 1) the most
// (lowest index wins ties); the sample taken from it is that source's running counter modulo its length.
inline void build_blend_index(const double* weights, const int64_t* lengths, int64_t n, int64_t size,
                              int32_t* dataset_index, int64_t* sample_index) {
  double total = 0;
  for (int64_t k = 0; k < n; ++k) total += weights[k];
  std::vector<int64_t> counts(static_cast<size_t>(n), 0);
  for (int64_t i = 0; i < size; ++i) {
    int64_t best = 0;
    double best_err = -1e300;
    for (int64_t k = 0; k < n; ++k) {
      const double err = (weights[k] / total) * static_cast<double>(i + 1) - static_cast<double>(counts[k]);
      if (err > best_err) {
        best_err = err;
        best = k;
      }
    }
    dataset_index[i] = static_cast<int32_t>(best);
    sample_index[i] = lengths[best] > 0 ? counts[best] % lengths[best] : 0;
    ++counts[best];
  }
}

// ------------------------------------------------------------------------------------ mmap token reader
// Read-only mapping of one or more token files that logically form one array of `dtype_bytes`-sized tokens.
class MMapTokens {
 public:
  MMapTokens(const std::vector<std::string>& paths, int64_t dtype_bytes) : dtype_bytes_(dtype_bytes) {
    int64_t start = 0;
    for (const auto& p : paths) {
      int fd = ::open(p.c_str(), O_RDONLY);
      if (fd < 0) {
        unmap_all();
        throw std::runtime_error("cannot open " + p);
      }
      struct stat st;
      ::fstat(fd, &st);
      void* addr = st.st_size > 0 ? ::mmap(nullptr, st.st_size, PROT_READ, MAP_PRIVATE, fd, 0) : nullptr;
      ::close(fd);
      if (addr == MAP_FAILED) {
        unmap_all();
        throw std::runtime_error("mmap failed for " + p);
      }
      parts_.push_back({static_cast<const char*>(addr), static_cast<int64_t>(st.st_size), start});
      start += st.st_size;
    }
    total_bytes_ = start;
  }
  ~MMapTokens() { unmap_all(); }
  MMapTokens(const MMapTokens&) = delete;
  MMapTokens& operator=(const MMapTokens&) = delete;

  // Copy the token spans [byte_offsets[i], byte_offsets[i] + counts[i]*dtype_bytes) back to back into `dst`
  // (`out_len` int32 values, zero-filled beyond the spans).
  void gather(const int64_t* byte_offsets, const int64_t* counts, int64_t n_spans, int32_t* dst, int64_t out_len) const {
    for (int64_t i = 0; i < out_len; ++i) dst[i] = 0;
    int64_t pos = 0;
    for (int64_t i = 0; i < n_spans; ++i) {
      int64_t b = byte_offsets[i];
      for (int64_t t = 0; t < counts[i] && pos < out_len; ++t, ++pos, b += dtype_bytes_) dst[pos] = read_token(b);
    }
  }
  int64_t total_bytes() const { return total_bytes_; }

 private:
  struct Part {
    const char* addr;
    int64_t size;
    int64_t start;
  };
  void unmap_all() {
    for (auto& p : parts_)
      if (p.addr) ::munmap(const_cast<char*>(p.addr), p.size);
    parts_.clear();
  }
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
      case 1: { uint8_t v; std::memcpy(&v, p, 1); return v; }
      case 2: { uint16_t v; std::memcpy(&v, p, 2); return v; }
      case 4: { int32_t v; std::memcpy(&v, p, 4); return v; }
      default: { int64_t v; std::memcpy(&v, p, 8); return static_cast<int32_t>(v); }
    }
  }
  std::vector<Part> parts_;
  int64_t dtype_bytes_;
  int64_t total_bytes_ = 0;
};

}  // namespace mtio
