// Native token-shard loader (see loader.h).  Shard format: 256 little-endian int32 header words
// {20240520, 1, num_tokens, 0...} followed by num_tokens little-endian uint16 ids; the file size must match exactly
// (parameter-golf-rs/crates/pg-data/src/shard.rs:6-17,36-77).
#include "loader.h"

#include <cuda_runtime.h>
#include <fcntl.h>
#include <string.h>
#include <sys/mman.h>
#include <sys/stat.h>
#include <unistd.h>

#include <stdexcept>

namespace pgb {

namespace {
constexpr int kMagic = 20240520, kVersion = 1;
constexpr size_t kHeaderBytes = 1024;

ShardMap map_shard(const std::string& path) {
  const int fd = ::open(path.c_str(), O_RDONLY);
  if (fd < 0) throw std::runtime_error(path + ": cannot open");
  struct stat st;
  if (fstat(fd, &st) != 0) { ::close(fd); throw std::runtime_error(path + ": cannot stat"); }
  const size_t size = (size_t)st.st_size;
  if (size < kHeaderBytes) { ::close(fd); throw std::runtime_error(path + ": shorter than the 1024-byte header"); }
  void* base = mmap(nullptr, size, PROT_READ, MAP_PRIVATE, fd, 0);
  ::close(fd);
  if (base == MAP_FAILED) throw std::runtime_error(path + ": mmap failed");
  const int32_t* h = static_cast<const int32_t*>(base);
  std::string err;
  if (h[0] != kMagic) err = path + ": bad magic " + std::to_string(h[0]);
  else if (h[1] != kVersion) err = path + ": unsupported version " + std::to_string(h[1]);
  else if (h[2] < 0 || size != kHeaderBytes + 2 * (size_t)h[2])
    err = path + ": size " + std::to_string(size) + " does not match header token count " + std::to_string(h[2]);
  if (!err.empty()) { munmap(base, size); throw std::runtime_error(err); }
  madvise(base, size, MADV_SEQUENTIAL);
  ShardMap m;
  m.base = base;
  m.bytes = size;
  m.count = h[2];
  m.tokens = reinterpret_cast<const uint16_t*>(static_cast<const char*>(base) + kHeaderBytes);
  return m;
}

void unmap(ShardMap& m) {
  if (m.base) munmap(m.base, m.bytes);
  m = ShardMap();
}
}  // namespace

ShardLoader::ShardLoader(std::vector<std::string> files, int rank, int world) : files_(std::move(files)), rank_(rank), world_(world) {
  if (files_.empty()) throw std::runtime_error("no shard files");
  if (rank < 0 || rank >= world) throw std::runtime_error("rank must be in [0, world_size)");
  open(0);
}

ShardLoader::~ShardLoader() {
  stop_prefetch();
  unmap(cur_);
}

void ShardLoader::open(int idx) {
  unmap(cur_);
  file_idx_ = idx % (int)files_.size();
  cur_ = map_shard(files_[file_idx_]);
  pos_ = 0;
}

void ShardLoader::restore(int file_idx, long long pos) {
  open(file_idx);
  pos_ = pos;
}

void ShardLoader::take(uint16_t* out, long long n) {
  long long done = 0;
  size_t empties = 0;
  while (done < n) {
    const long long avail = cur_.count - pos_;
    if (avail <= 0) {
      open(file_idx_ + 1);
      if (++empties > files_.size()) throw std::runtime_error("all shards are empty");
      continue;
    }
    empties = 0;
    const long long k = std::min(n - done, avail);
    memcpy(out + done, cur_.tokens + pos_, (size_t)k * 2);
    pos_ += k;
    done += k;
  }
}

void ShardLoader::skip(long long n) {
  size_t empties = 0;
  while (n > 0) {
    const long long avail = cur_.count - pos_;
    if (avail <= 0) {
      open(file_idx_ + 1);
      if (++empties > files_.size()) throw std::runtime_error("all shards are empty");
      continue;
    }
    empties = 0;
    const long long k = std::min(n, avail);
    pos_ += k;
    n -= k;
  }
}

void ShardLoader::next_span(uint16_t* out, long long global_tokens, int grad_accum) {
  const long long span = global_tokens / ((long long)world_ * grad_accum) + 1;
  skip((long long)rank_ * span);
  take(out, span);
  skip((long long)(world_ - 1 - rank_) * span);
}

void ShardLoader::start_prefetch(long long global_tokens, int grad_accum, int depth, int keep) {
  stop_prefetch();
  if (keep < 1) keep = 1;
  if (depth < keep + 1) depth = keep + 1;
  keep_ = keep;
  global_ = global_tokens;
  accum_ = grad_accum;
  span_ = global_tokens / ((long long)world_ * grad_accum) + 1;
  const size_t bytes = ((size_t)span_ * 2 + 255) / 256 * 256;
  ring_.assign(depth, nullptr);
  ring_file_.assign(depth, 0);
  ring_pos_.assign(depth, 0);
  int ndev = 0;
  pinned_ = cudaGetDeviceCount(&ndev) == cudaSuccess && ndev > 0;
  if (!pinned_) cudaGetLastError();
  for (int i = 0; i < depth; ++i) {
    void* p = nullptr;
    if (pinned_ && cudaHostAlloc(&p, bytes, cudaHostAllocDefault) != cudaSuccess) {
      cudaGetLastError();
      pinned_ = false;
      for (int j = 0; j < i; ++j) { cudaFreeHost(ring_[j]); ring_[j] = nullptr; }
      i = -1;                                          // start over with plain memory
      continue;
    }
    if (!pinned_) p = ::operator new(bytes);
    ring_[i] = static_cast<uint16_t*>(p);
  }
  produced_ = consumed_ = 0;
  stop_ = false;
  error_.clear();
  running_ = true;
  thread_ = std::thread(&ShardLoader::worker, this);
}

void ShardLoader::worker() {
  const long long depth = (long long)ring_.size();
  for (;;) {
    {
      std::unique_lock<std::mutex> lk(mu_);
      // the slot being filled must not be one of the `keep_` spans the consumer may still read
      cv_.wait(lk, [&] { return stop_ || produced_ - consumed_ < depth - keep_; });
      if (stop_) return;
    }
    const int slot = (int)(produced_ % depth);
    try {
      next_span(ring_[slot], global_, accum_);
    } catch (const std::exception& e) {
      std::lock_guard<std::mutex> lk(mu_);
      error_ = e.what();
      stop_ = true;
      cv_.notify_all();
      return;
    }
    {
      std::lock_guard<std::mutex> lk(mu_);
      ring_file_[slot] = file_idx_;
      ring_pos_[slot] = pos_;
      ++produced_;
    }
    cv_.notify_all();
  }
}

const uint16_t* ShardLoader::next_prefetched(int* file_idx_after, long long* pos_after) {
  if (!running_) throw std::runtime_error("prefetch is not running");
  std::unique_lock<std::mutex> lk(mu_);
  cv_.wait(lk, [&] { return produced_ > consumed_ || !error_.empty(); });
  if (produced_ <= consumed_) throw std::runtime_error("shard prefetch failed: " + error_);
  const int slot = (int)(consumed_ % (long long)ring_.size());
  ++consumed_;
  if (file_idx_after) *file_idx_after = ring_file_[slot];
  if (pos_after) *pos_after = ring_pos_[slot];
  lk.unlock();
  cv_.notify_all();
  return ring_[slot];
}

void ShardLoader::stop_prefetch() {
  if (running_) {
    {
      std::lock_guard<std::mutex> lk(mu_);
      stop_ = true;
    }
    cv_.notify_all();
    if (thread_.joinable()) thread_.join();
    running_ = false;
  }
  for (auto*& p : ring_) {
    if (p) {
      if (pinned_) cudaFreeHost(p); else ::operator delete(p);
      p = nullptr;
    }
  }
  ring_.clear();
}

}  // namespace pgb
