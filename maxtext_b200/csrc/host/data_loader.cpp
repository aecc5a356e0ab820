// Native batch producer for token files: memory-mapped readers, sequence packing and a background thread that keeps a
// bounded queue of ready [batch, seq] tensors, so the training loop's `next()` is a memcpy into pinned memory.
//
// The role of the reference's Grain pipeline workers (src/maxtext/input_pipeline/grain_data_processing.py,
// olmo_grain_data_processing.py): pre-tokenized files -> documents -> packed rows (inputs, targets shifted by one,
// segment ids, positions) -> per-host batches, with a position that a checkpoint can store and seek back to.
//
// Files are flat int32 token streams (raw .bin, or .npy with a v1/v2 header); a document ends at every `eos` token.
// Documents are dealt round-robin to the data-parallel ranks (document d goes to rank d % world). A row is filled with
// consecutive documents of the rank until the next one does not fit (it then starts the next row); documents longer
// than seq + 1 tokens are cut into pieces of that length. Everything is deterministic in (files, seq, batch, rank, world).
#include <torch/extension.h>

#include <fcntl.h>
#include <sys/mman.h>
#include <sys/stat.h>
#include <unistd.h>

#include <condition_variable>
#include <cstring>
#include <deque>
#include <mutex>
#include <string>
#include <thread>
#include <vector>

namespace {

struct Mapped {
  const int32_t* data = nullptr;
  int64_t n = 0;
  void* base = nullptr;
  size_t bytes = 0;
};

Mapped map_file(const std::string& path) {
  Mapped m;
  int fd = ::open(path.c_str(), O_RDONLY);
  TORCH_CHECK(fd >= 0, "cannot open ", path);
  struct stat st;
  TORCH_CHECK(::fstat(fd, &st) == 0, "cannot stat ", path);
  m.bytes = (size_t)st.st_size;
  m.base = m.bytes ? ::mmap(nullptr, m.bytes, PROT_READ, MAP_PRIVATE, fd, 0) : nullptr;
  ::close(fd);
  TORCH_CHECK(m.bytes == 0 || m.base != MAP_FAILED, "cannot map ", path);
  size_t off = 0;
  const unsigned char* b = static_cast<const unsigned char*>(m.base);
  if (m.bytes >= 10 && std::memcmp(b, "\x93NUMPY", 6) == 0) {            // .npy: magic, version, header length, header
    const int major = b[6];
    const size_t hlen = major == 1 ? (size_t)b[8] | ((size_t)b[9] << 8)
                                   : (size_t)b[8] | ((size_t)b[9] << 8) | ((size_t)b[10] << 16) | ((size_t)b[11] << 24);
    off = (major == 1 ? 10 : 12) + hlen;
    const std::string header(reinterpret_cast<const char*>(b) + (major == 1 ? 10 : 12), hlen);
    TORCH_CHECK(header.find("<i4") != std::string::npos || header.find("|i4") != std::string::npos, path, ": expected int32 tokens");
  }
  m.data = reinterpret_cast<const int32_t*>(b + off);
  m.n = (int64_t)((m.bytes - off) / sizeof(int32_t));
  return m;
}

struct Cursor {
  int64_t file = 0, pos = 0, doc = 0, epoch = 0;
};

struct Batch {
  std::vector<int32_t> inputs, targets, segments, positions;
  Cursor after;                      // where the stream stands once this batch has been produced
};

}  // namespace

class TokenLoader {
 public:
  TokenLoader(std::vector<std::string> paths, int64_t seq, int64_t batch, int64_t eos, int64_t rank, int64_t world, int64_t depth)
      : seq_(seq), batch_(batch), eos_((int32_t)eos), rank_(rank), world_(world), depth_(depth > 0 ? depth : 2) {
    TORCH_CHECK(!paths.empty(), "no token files");
    TORCH_CHECK(seq > 0 && batch > 0 && world > 0 && rank >= 0 && rank < world, "bad loader geometry");
    for (auto& p : paths) files_.push_back(map_file(p));
    int64_t total = 0;
    for (auto& f : files_) total += f.n;
    TORCH_CHECK(total > 1, "token files are empty");
    const int32_t* p0 = nullptr;
    int64_t l0 = 0;
    Cursor a0;
    if (!peek(cur_, p0, l0, a0))
      throw std::runtime_error("rank " + std::to_string(rank_) + " of " + std::to_string(world_) + " finds no document of two or more tokens");
    start();
  }

  ~TokenLoader() {
    stop();
    for (auto& f : files_)
      if (f.base && f.bytes) ::munmap(f.base, f.bytes);
  }

  // Copies the next batch into the four [batch, seq] int32 CPU tensors (pinned or not).
  void next(torch::Tensor inputs, torch::Tensor targets, torch::Tensor segments, torch::Tensor positions) {
    const int64_t n = batch_ * seq_;
    for (auto* t : {&inputs, &targets, &segments, &positions})
      TORCH_CHECK(t->device().is_cpu() && t->scalar_type() == torch::kInt32 && t->is_contiguous() && t->numel() == n,
                  "next() wants contiguous int32 CPU tensors of batch x seq elements");
    Batch b;
    {
      pybind11::gil_scoped_release release;
      std::unique_lock<std::mutex> lk(mu_);
      cv_ready_.wait(lk, [&] { return !ready_.empty(); });
      b = std::move(ready_.front());
      ready_.pop_front();
      handed_ = b.after;
      cv_space_.notify_one();
    }
    std::memcpy(inputs.data_ptr<int32_t>(), b.inputs.data(), n * sizeof(int32_t));
    std::memcpy(targets.data_ptr<int32_t>(), b.targets.data(), n * sizeof(int32_t));
    std::memcpy(segments.data_ptr<int32_t>(), b.segments.data(), n * sizeof(int32_t));
    std::memcpy(positions.data_ptr<int32_t>(), b.positions.data(), n * sizeof(int32_t));
  }

  // Stream position after the last batch handed out: (file, offset, document index, epoch).
  std::vector<int64_t> state() {
    std::lock_guard<std::mutex> lk(mu_);
    return {handed_.file, handed_.pos, handed_.doc, handed_.epoch};
  }

  void seek(std::vector<int64_t> s) {
    TORCH_CHECK(s.size() == 4, "state has four numbers");
    stop();
    cur_.file = s[0], cur_.pos = s[1], cur_.doc = s[2], cur_.epoch = s[3];
    TORCH_CHECK(cur_.file >= 0 && cur_.file < (int64_t)files_.size() && cur_.pos >= 0 && cur_.pos <= files_[cur_.file].n, "state out of range");
    handed_ = cur_;
    ready_.clear();
    start();
  }

 private:
  // The next piece of this rank's documents at cursor `c`: [begin, begin + len) of file c.file, and the cursor after it.
  // A piece has at most seq + 1 tokens; consecutive pieces of a long document overlap by one token (the last target of one
  // is the first input of the next).
  bool peek(const Cursor& c, const int32_t*& begin, int64_t& len, Cursor& after) {
    Cursor k = c;
    for (int64_t guard = 0; guard < (int64_t)files_.size() * 2 + 4;) {
      const Mapped& f = files_[k.file];
      if (k.pos >= f.n) {                                   // next file (or next epoch)
        k.pos = 0;
        if (++k.file == (int64_t)files_.size()) k.file = 0, k.doc = 0, ++k.epoch;
        ++guard;
        continue;
      }
      int64_t end = k.pos;
      while (end < f.n && f.data[end] != eos_) ++end;
      const bool closed = end < f.n;                        // the document ends with an eos token (kept as its last token)
      const int64_t doc_len = end - k.pos + (closed ? 1 : 0);
      const bool mine = k.doc % world_ == rank_;
      if (!mine || doc_len < 2) {
        k.pos += doc_len;
        ++k.doc;
        continue;
      }
      begin = f.data + k.pos;
      if (doc_len > seq_ + 1) {
        len = seq_ + 1;
        k.pos += seq_;                                      // stay inside the document: same index, same rank
      } else {
        len = doc_len;
        k.pos += doc_len;
        ++k.doc;
      }
      after = k;
      return true;
    }
    return false;                                           // this rank has no usable document in any file
  }

  Batch make_batch() {
    Batch b;
    const int64_t n = batch_ * seq_;
    b.inputs.assign(n, 0), b.targets.assign(n, 0), b.segments.assign(n, 0), b.positions.assign(n, 0);
    for (int64_t r = 0; r < batch_; ++r) {
      int64_t used = 0;
      int32_t seg = 0;
      while (used < seq_) {
        const int32_t* p;
        int64_t len;
        Cursor after;
        if (!peek(cur_, p, len, after)) {                    // cannot happen: the constructor found one
          b.after = cur_;
          return b;
        }
        const int64_t need = len - 1;
        if (need > seq_ - used) {
          if (used > 0) break;                              // does not fit: it opens the next row
        }
        const int64_t take = need < seq_ - used ? need : seq_ - used;
        ++seg;
        int32_t* in = b.inputs.data() + r * seq_ + used;
        int32_t* tg = b.targets.data() + r * seq_ + used;
        int32_t* sg = b.segments.data() + r * seq_ + used;
        int32_t* ps = b.positions.data() + r * seq_ + used;
        for (int64_t i = 0; i < take; ++i) in[i] = p[i], tg[i] = p[i + 1], sg[i] = seg, ps[i] = (int32_t)i;
        used += take;
        cur_ = after;
      }
    }
    b.after = cur_;
    return b;
  }

  void start() {
    stop_ = false;
    worker_ = std::thread([this] {
      for (;;) {
        Batch b = make_batch();
        std::unique_lock<std::mutex> lk(mu_);
        cv_space_.wait(lk, [&] { return stop_ || (int64_t)ready_.size() < depth_; });
        if (stop_) return;
        ready_.push_back(std::move(b));
        cv_ready_.notify_one();
      }
    });
  }

  void stop() {
    {
      std::lock_guard<std::mutex> lk(mu_);
      stop_ = true;
    }
    cv_space_.notify_all();
    if (worker_.joinable()) worker_.join();
  }

  std::vector<Mapped> files_;
  int64_t seq_, batch_;
  int32_t eos_;
  int64_t rank_, world_, depth_;
  Cursor cur_, handed_;
  std::deque<Batch> ready_;
  std::mutex mu_;
  std::condition_variable cv_ready_, cv_space_;
  std::thread worker_;
  bool stop_ = false;
};

PYBIND11_MODULE(TORCH_EXTENSION_NAME, m) {
  pybind11::class_<TokenLoader>(m, "TokenLoader")
      .def(pybind11::init<std::vector<std::string>, int64_t, int64_t, int64_t, int64_t, int64_t, int64_t>(), pybind11::arg("paths"),
           pybind11::arg("seq"), pybind11::arg("batch"), pybind11::arg("eos"), pybind11::arg("rank") = 0, pybind11::arg("world") = 1,
           pybind11::arg("depth") = 2)
      .def("next", &TokenLoader::next)
      .def("state", &TokenLoader::state)
      .def("seek", &TokenLoader::seek);
}
