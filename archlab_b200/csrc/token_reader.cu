// Native prefetching reader for raw-int32 token parts (host code only).
//
// Deterministic addressing identical to the Python statement in archlab_b200/data/token_batches.py
// (and to the reference iterator, src/archlab/megatron/token_batches.py:12-120): batch index b reads
// part (b mod P) at token offset (b div P) * batch * seq, cyclically, `batch * seq + 1` tokens, widened
// to int64.  A worker thread keeps one batch ahead of the consumer so that file reads and the
// int32 -> int64 widening overlap the training step; the consumer copies the finished batch into a
// caller-provided (pinned) buffer.
#include <atomic>
#include <condition_variable>
#include <cstdint>
#include <cstring>
#include <fcntl.h>
#include <mutex>
#include <string>
#include <sys/mman.h>
#include <sys/stat.h>
#include <thread>
#include <unistd.h>
#include <vector>

namespace {

struct Part {
  const int32_t* data = nullptr;
  size_t tokens = 0;
  size_t bytes = 0;
};

struct Reader {
  std::vector<Part> parts;
  long long batch = 0, seq = 0, start_batch = 0, repeat_window = 0;
  long long next_batch = 0;       // batch index the consumer will receive next
  std::vector<int64_t> ready;     // prefetched batch (flat, batch*seq + 1 tokens)
  long long ready_index = -1;
  bool stop = false;
  std::mutex mu;
  std::condition_variable cv;
  std::thread worker;

  long long source_index(long long b) const {
    if (repeat_window <= 0) return b;
    return start_batch + ((b - start_batch) % repeat_window);
  }
  void fill(long long b, int64_t* dst) const {
    const long long src = source_index(b);
    const Part& p = parts[size_t(src % (long long)parts.size())];
    const size_t flat = size_t(batch * seq);
    size_t pos = size_t((src / (long long)parts.size()) * (long long)flat) % p.tokens;
    for (size_t i = 0; i < flat + 1; ++i) {
      dst[i] = (int64_t)p.data[pos];
      if (++pos == p.tokens) pos = 0;
    }
  }
  void run() {
    std::vector<int64_t> scratch(size_t(batch * seq + 1));
    std::unique_lock<std::mutex> lk(mu);
    while (!stop) {
      if (ready_index == next_batch) {       // already prefetched; wait until it is consumed
        cv.wait(lk);
        continue;
      }
      const long long want = next_batch;
      lk.unlock();
      fill(want, scratch.data());
      lk.lock();
      if (want == next_batch) {
        ready.swap(scratch);
        ready_index = want;
        cv.notify_all();
      }
    }
  }
};

}  // namespace

extern "C" void* nga_reader_open(const char* const* bin_paths, int n_parts, long long batch, long long seq,
                                 long long start_batch, long long repeat_window) {
  if (n_parts <= 0 || batch <= 0 || seq <= 0 || start_batch < 0) return nullptr;
  Reader* r = new Reader();
  r->batch = batch; r->seq = seq; r->start_batch = start_batch; r->repeat_window = repeat_window;
  r->next_batch = start_batch;
  for (int i = 0; i < n_parts; ++i) {
    int fd = ::open(bin_paths[i], O_RDONLY);
    if (fd < 0) { delete r; return nullptr; }
    struct stat st;
    if (fstat(fd, &st) != 0 || st.st_size < (off_t)((seq + 1) * 4)) { ::close(fd); delete r; return nullptr; }
    void* m = mmap(nullptr, (size_t)st.st_size, PROT_READ, MAP_PRIVATE, fd, 0);
    ::close(fd);
    if (m == MAP_FAILED) { delete r; return nullptr; }
    Part p;
    p.data = static_cast<const int32_t*>(m);
    p.bytes = (size_t)st.st_size;
    p.tokens = p.bytes / 4;
    r->parts.push_back(p);
  }
  r->ready.resize(size_t(batch * seq + 1));
  r->worker = std::thread([r] { r->run(); });
  return r;
}

// Copies batch `next` (batch*seq + 1 int64 tokens) into dst and advances; returns its index.
extern "C" long long nga_reader_next(void* handle, int64_t* dst) {
  Reader* r = static_cast<Reader*>(handle);
  std::unique_lock<std::mutex> lk(r->mu);
  r->cv.wait(lk, [r] { return r->ready_index == r->next_batch; });
  std::memcpy(dst, r->ready.data(), sizeof(int64_t) * size_t(r->batch * r->seq + 1));
  const long long idx = r->next_batch;
  r->next_batch += 1;
  r->cv.notify_all();
  return idx;
}

extern "C" void nga_reader_close(void* handle) {
  Reader* r = static_cast<Reader*>(handle);
  {
    std::lock_guard<std::mutex> lk(r->mu);
    r->stop = true;
    r->cv.notify_all();
  }
  if (r->worker.joinable()) r->worker.join();
  for (auto& p : r->parts) munmap(const_cast<int32_t*>(p.data), p.bytes);
  delete r;
}
