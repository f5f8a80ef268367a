// Native positioned-read engine for expert streaming and checkpoint loading.
//
// A fixed pool of worker threads executes read requests (file, offset, length -> destination
// pointer, normally inside a registered pinned slab).  A request whose offset, length and
// destination are all 4 KiB aligned is served through an O_DIRECT descriptor (no page-cache copy);
// anything else goes through a buffered descriptor.  Completions are collected by polling
// (`fb_reader_poll`) or by blocking with a timeout (`fb_reader_wait`); every request carries the
// caller's 64-bit tag.  Requests can be cancelled while still queued.
//
// Plays the role of the reference's io_uring direct reader
// (crates/ferrule-model/src/moe/io_uring_reader.rs:31-230 registered buffers, :612-2030 submission
// and completion pump, :2034-2260 tickets and cancellation) with a thread pool instead of a ring:
// the container this runs in does not expose io_uring.
#include <fcntl.h>
#include <unistd.h>

#include <atomic>
#include <cerrno>
#include <chrono>
#include <condition_variable>
#include <cstdint>
#include <cstring>
#include <deque>
#include <mutex>
#include <string>
#include <thread>
#include <unordered_map>
#include <vector>

namespace {

constexpr uint64_t kAlign = 4096;

struct Request {
  uint64_t tag;
  std::string path;
  uint64_t offset;
  uint64_t length;
  char* dst;
};

struct Completion {
  uint64_t tag;
  int64_t result;  // bytes read, or -errno, or -ECANCELED
};

class Reader {
 public:
  explicit Reader(int threads) {
    if (threads < 1) threads = 1;
    for (int i = 0; i < threads; ++i) workers_.emplace_back([this] { run(); });
  }
  ~Reader() {
    {
      std::lock_guard<std::mutex> l(mu_);
      stop_ = true;
    }
    cv_.notify_all();
    for (auto& t : workers_) t.join();
    for (auto& kv : fds_) ::close(kv.second);
  }
  void submit(Request r) {
    {
      std::lock_guard<std::mutex> l(mu_);
      queue_.push_back(std::move(r));
      ++submitted_;
    }
    cv_.notify_one();
  }
  bool cancel(uint64_t tag) {
    std::lock_guard<std::mutex> l(mu_);
    for (auto it = queue_.begin(); it != queue_.end(); ++it) {
      if (it->tag == tag) {
        queue_.erase(it);
        done_.push_back({tag, -ECANCELED});
        done_cv_.notify_all();
        return true;
      }
    }
    return false;
  }
  int poll(Completion* out, int max, int timeout_ms) {
    std::unique_lock<std::mutex> l(mu_);
    if (done_.empty() && timeout_ms > 0)
      done_cv_.wait_for(l, std::chrono::milliseconds(timeout_ms), [this] { return !done_.empty(); });
    int n = 0;
    while (n < max && !done_.empty()) {
      out[n++] = done_.front();
      done_.pop_front();
    }
    return n;
  }
  void stats(uint64_t* s) {
    std::lock_guard<std::mutex> l(mu_);
    s[0] = submitted_;
    s[1] = completed_;
    s[2] = bytes_;
    s[3] = direct_reads_;
    s[4] = queue_.size();
  }

 private:
  int fd_for(const std::string& path, bool direct) {
    const std::string key = (direct ? "D:" : "B:") + path;
    {
      std::lock_guard<std::mutex> l(fd_mu_);
      auto it = fds_.find(key);
      if (it != fds_.end()) return it->second;
    }
    int flags = O_RDONLY | O_CLOEXEC;
#ifdef O_DIRECT
    if (direct) flags |= O_DIRECT;
#endif
    int fd = ::open(path.c_str(), flags);
    if (fd < 0 && direct) return -1;  // file system without O_DIRECT: caller falls back
    if (fd < 0) return -errno;
    std::lock_guard<std::mutex> l(fd_mu_);
    auto ins = fds_.emplace(key, fd);
    if (!ins.second) {
      ::close(fd);
      return ins.first->second;
    }
    return fd;
  }
  int64_t do_read(const Request& r, bool* used_direct) {
    const bool aligned = (r.offset % kAlign == 0) && (r.length % kAlign == 0) &&
                         (reinterpret_cast<uintptr_t>(r.dst) % kAlign == 0);
    int fd = -1;
    *used_direct = false;
    if (aligned) {
      fd = fd_for(r.path, true);
      *used_direct = fd >= 0;
    }
    if (fd < 0) fd = fd_for(r.path, false);
    if (fd < 0) return fd;
    uint64_t got = 0;
    while (got < r.length) {
      ssize_t n = ::pread(fd, r.dst + got, r.length - got, static_cast<off_t>(r.offset + got));
      if (n < 0) {
        if (errno == EINTR) continue;
        return -errno;
      }
      if (n == 0) break;  // end of file: short read, reported as such
      got += static_cast<uint64_t>(n);
    }
    return static_cast<int64_t>(got);
  }
  void run() {
    for (;;) {
      Request r;
      {
        std::unique_lock<std::mutex> l(mu_);
        cv_.wait(l, [this] { return stop_ || !queue_.empty(); });
        if (stop_ && queue_.empty()) return;
        r = std::move(queue_.front());
        queue_.pop_front();
      }
      bool direct = false;
      const int64_t res = do_read(r, &direct);
      {
        std::lock_guard<std::mutex> l(mu_);
        done_.push_back({r.tag, res});
        ++completed_;
        if (res > 0) bytes_ += static_cast<uint64_t>(res);
        if (direct) ++direct_reads_;
      }
      done_cv_.notify_all();
    }
  }

  std::mutex mu_, fd_mu_;
  std::condition_variable cv_, done_cv_;
  std::deque<Request> queue_;
  std::deque<Completion> done_;
  std::vector<std::thread> workers_;
  std::unordered_map<std::string, int> fds_;
  bool stop_ = false;
  uint64_t submitted_ = 0, completed_ = 0, bytes_ = 0, direct_reads_ = 0;
};

}  // namespace

extern "C" {

void* fb_reader_create(int threads) { return new Reader(threads); }

void fb_reader_destroy(void* h) { delete static_cast<Reader*>(h); }

int fb_reader_submit(void* h, unsigned long long tag, const char* path, unsigned long long offset,
                     unsigned long long length, void* dst) {
  if (!h || !path || !dst || length == 0) return 1;
  static_cast<Reader*>(h)->submit({tag, path, offset, length, static_cast<char*>(dst)});
  return 0;
}

int fb_reader_cancel(void* h, unsigned long long tag) {
  return h && static_cast<Reader*>(h)->cancel(tag) ? 1 : 0;
}

// tags_out / results_out hold up to `max` entries; returns the number of completions written.
int fb_reader_poll(void* h, unsigned long long* tags_out, long long* results_out, int max, int timeout_ms) {
  if (!h || max <= 0) return 0;
  std::vector<Completion> buf(static_cast<size_t>(max));
  const int n = static_cast<Reader*>(h)->poll(buf.data(), max, timeout_ms);
  for (int i = 0; i < n; ++i) {
    tags_out[i] = buf[i].tag;
    results_out[i] = buf[i].result;
  }
  return n;
}

// out[5] = {submitted, completed, bytes, direct_reads, queued}
void fb_reader_stats(void* h, unsigned long long* out) {
  uint64_t s[5] = {0, 0, 0, 0, 0};
  if (h) static_cast<Reader*>(h)->stats(s);
  for (int i = 0; i < 5; ++i) out[i] = s[i];
}

}  // extern "C"
