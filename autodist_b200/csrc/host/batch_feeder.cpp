// Background batch feeder: worker threads assemble (optionally shuffled) batches of fixed-size records from a
// memory-mapped file into a ring of caller-provided buffers - pinned host tensors in practice, so that the session can
// start the upload of batch i + 1 while step i runs. The counterpart of the input pipelines the reference builds from
// tf.data (interleave -> shuffle -> batch -> prefetch, examples/benchmark/utils/input_pipeline.py:82-131 and
// imagenet_preprocessing.py:242-316), reduced to what a training loop over pre-processed records needs.
//
// Records are `record_bytes` long and hold the fields back to back; a batch buffer holds every field as one
// contiguous block ([batch, field bytes]), so each field is a contiguous tensor on the Python side. With `world`
// replicas every epoch is one permutation of all records (seeded, the same on every rank) of which rank r takes
// elements r, r + world, ...; every rank sees the same number of batches.
//
// Order is fixed: batch b lands in slot b % depth and is handed out in order b = 0, 1, 2, ... whatever the number of
// worker threads; a slot is refilled only after the consumer released it.
#include <fcntl.h>
#include <pybind11/pybind11.h>
#include <pybind11/stl.h>
#include <sys/mman.h>
#include <sys/stat.h>
#include <unistd.h>

#include <algorithm>
#include <condition_variable>
#include <cstdint>
#include <cstring>
#include <map>
#include <memory>
#include <mutex>
#include <numeric>
#include <random>
#include <stdexcept>
#include <string>
#include <thread>
#include <vector>

namespace py = pybind11;

namespace {

class BatchFeeder {
 public:
  BatchFeeder(const std::string& path, int64_t record_bytes, std::vector<std::pair<int64_t, int64_t>> fields, int64_t batch,
              std::vector<uint64_t> slot_ptrs, int workers, bool shuffle, uint64_t seed, bool drop_last, int64_t rank, int64_t world,
              int64_t epochs)
      : record_bytes_(record_bytes), fields_(std::move(fields)), batch_(batch), shuffle_(shuffle), seed_(seed), rank_(rank), world_(world) {
    if (record_bytes <= 0 || batch <= 0 || world <= 0 || rank < 0 || rank >= world || slot_ptrs.empty())
      throw std::invalid_argument("batch feeder: bad sizes");
    int64_t covered = 0;
    for (const auto& f : fields_) {
      if (f.first < 0 || f.second <= 0 || f.first + f.second > record_bytes) throw std::invalid_argument("batch feeder: a field leaves the record");
      covered += f.second;
    }
    batch_bytes_ = covered * batch;
    fd_ = ::open(path.c_str(), O_RDONLY);
    if (fd_ < 0) throw std::runtime_error("batch feeder: cannot open " + path);
    struct stat st;
    if (::fstat(fd_, &st) != 0 || st.st_size < record_bytes) {
      ::close(fd_);
      throw std::runtime_error("batch feeder: " + path + " holds no complete record");
    }
    file_bytes_ = (size_t)st.st_size;
    void* p = ::mmap(nullptr, file_bytes_, PROT_READ, MAP_PRIVATE, fd_, 0);
    if (p == MAP_FAILED) {
      ::close(fd_);
      throw std::runtime_error("batch feeder: mmap failed for " + path);
    }
    base_ = static_cast<const uint8_t*>(p);
    records_ = (int64_t)(file_bytes_ / (size_t)record_bytes);
    per_rank_ = records_ / world;
    if (per_rank_ == 0) {
      cleanup();
      throw std::runtime_error("batch feeder: fewer records than replicas");
    }
    batches_per_epoch_ = drop_last ? per_rank_ / batch : (per_rank_ + batch - 1) / batch;
    if (batches_per_epoch_ == 0) {
      cleanup();
      throw std::runtime_error("batch feeder: fewer records per replica than one batch");
    }
    total_ = epochs < 0 ? -1 : epochs * batches_per_epoch_;
    depth_ = (int64_t)slot_ptrs.size();
    for (uint64_t s : slot_ptrs) slots_.push_back(reinterpret_cast<uint8_t*>(s));
    slot_batch_.assign(depth_, kFree);
    slot_rows_.assign(depth_, 0);
    slot_next_.resize(depth_);
    std::iota(slot_next_.begin(), slot_next_.end(), (int64_t)0);
    const int n = std::max(1, std::min<int>(workers, (int)depth_));
    for (int i = 0; i < n; ++i) threads_.emplace_back([this] { work(); });
  }

  ~BatchFeeder() { close(); }

  void close() {
    {
      std::lock_guard<std::mutex> g(mu_);
      if (stop_) return;
      stop_ = true;
    }
    cv_.notify_all();
    for (auto& t : threads_)
      if (t.joinable()) t.join();
    cleanup();
  }

  // Slot of the next batch in order (blocks until a worker has filled it), or -1 after the last batch.
  int64_t next() {
    py::gil_scoped_release nogil;
    std::unique_lock<std::mutex> lk(mu_);
    if (total_ >= 0 && consumed_ >= total_) return -1;
    const int64_t slot = consumed_ % depth_;
    cv_.wait(lk, [&] { return stop_ || slot_batch_[slot] == consumed_; });
    if (stop_) return -1;
    ++consumed_;
    return slot;
  }

  int64_t rows(int64_t slot) {
    std::lock_guard<std::mutex> g(mu_);
    return slot_rows_.at(slot);
  }

  // The consumer is done with the slot (its upload has finished): a worker may fill it with the batch `depth` later.
  void release(int64_t slot) {
    {
      std::lock_guard<std::mutex> g(mu_);
      if (slot < 0 || slot >= depth_ || slot_batch_[slot] < 0) throw std::invalid_argument("batch feeder: slot is not handed out");
      slot_next_[slot] = slot_batch_[slot] + depth_;
      slot_batch_[slot] = kFree;
    }
    cv_.notify_all();
  }

  int64_t batches_per_epoch() const { return batches_per_epoch_; }
  int64_t records() const { return records_; }
  int64_t batch_bytes() const { return batch_bytes_; }

 private:
  static constexpr int64_t kFree = -1, kFilling = -2;

  void cleanup() {
    if (base_ != nullptr) ::munmap(const_cast<uint8_t*>(base_), file_bytes_);
    base_ = nullptr;
    if (fd_ >= 0) ::close(fd_);
    fd_ = -1;
  }

  std::shared_ptr<const std::vector<int64_t>> permutation(int64_t epoch) {
    std::lock_guard<std::mutex> g(perm_mu_);
    auto it = perms_.find(epoch);
    if (it != perms_.end()) return it->second;
    auto p = std::make_shared<std::vector<int64_t>>(records_);
    std::iota(p->begin(), p->end(), (int64_t)0);
    if (shuffle_) {
      std::mt19937_64 rng(seed_ * 0x9E3779B97F4A7C15ull + (uint64_t)epoch);
      for (int64_t i = records_ - 1; i > 0; --i) {             // Fisher-Yates with an explicit draw: the same on every platform
        const int64_t j = (int64_t)(rng() % (uint64_t)(i + 1));
        std::swap((*p)[i], (*p)[j]);
      }
    }
    while (perms_.size() >= 3) perms_.erase(perms_.begin());   // workers straddle at most two epochs
    perms_[epoch] = p;
    return p;
  }

  void work() {
    for (;;) {
      int64_t b, slot;
      {
        std::unique_lock<std::mutex> lk(mu_);
        if (stop_ || (total_ >= 0 && claimed_ >= total_)) return;
        b = claimed_++;
        slot = b % depth_;
        cv_.wait(lk, [&] { return stop_ || (slot_batch_[slot] == kFree && slot_next_[slot] == b); });
        if (stop_) return;
        slot_batch_[slot] = kFilling;
      }
      const int64_t epoch = b / batches_per_epoch_, k = b % batches_per_epoch_;
      const auto perm = permutation(epoch);
      const int64_t first = k * batch_, rows = std::min(batch_, per_rank_ - first);
      uint8_t* dst = slots_[slot];
      int64_t field_base = 0;
      for (const auto& f : fields_) {
        for (int64_t r = 0; r < rows; ++r) {
          const int64_t rec = (*perm)[(first + r) * world_ + rank_];
          std::memcpy(dst + field_base + r * f.second, base_ + rec * record_bytes_ + f.first, (size_t)f.second);
        }
        field_base += f.second * batch_;
      }
      {
        std::lock_guard<std::mutex> g(mu_);
        slot_rows_[slot] = rows;
        slot_batch_[slot] = b;
      }
      cv_.notify_all();
    }
  }

  int64_t record_bytes_;
  std::vector<std::pair<int64_t, int64_t>> fields_;      // (offset inside the record, bytes)
  int64_t batch_, batch_bytes_ = 0;
  bool shuffle_;
  uint64_t seed_;
  int64_t rank_, world_;
  int fd_ = -1;
  const uint8_t* base_ = nullptr;
  size_t file_bytes_ = 0;
  int64_t records_ = 0, per_rank_ = 0, batches_per_epoch_ = 0, total_ = 0, depth_ = 0;
  std::vector<uint8_t*> slots_;
  std::mutex mu_, perm_mu_;
  std::condition_variable cv_;
  std::vector<int64_t> slot_batch_, slot_rows_, slot_next_;
  int64_t claimed_ = 0, consumed_ = 0;
  bool stop_ = false;
  std::map<int64_t, std::shared_ptr<const std::vector<int64_t>>> perms_;
  std::vector<std::thread> threads_;
};

}  // namespace

void register_batch_feeder(py::module& m) {
  py::class_<BatchFeeder>(m, "BatchFeeder")
      .def(py::init<const std::string&, int64_t, std::vector<std::pair<int64_t, int64_t>>, int64_t, std::vector<uint64_t>, int, bool, uint64_t,
                    bool, int64_t, int64_t, int64_t>(),
           py::arg("path"), py::arg("record_bytes"), py::arg("fields"), py::arg("batch"), py::arg("slot_ptrs"), py::arg("workers") = 2,
           py::arg("shuffle") = true, py::arg("seed") = 0, py::arg("drop_last") = true, py::arg("rank") = 0, py::arg("world") = 1,
           py::arg("epochs") = 1)
      .def("next", &BatchFeeder::next)
      .def("rows", &BatchFeeder::rows)
      .def("release", &BatchFeeder::release)
      .def("close", &BatchFeeder::close)
      .def_property_readonly("batches_per_epoch", &BatchFeeder::batches_per_epoch)
      .def_property_readonly("records", &BatchFeeder::records)
      .def_property_readonly("batch_bytes", &BatchFeeder::batch_bytes);
}
