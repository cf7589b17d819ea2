// Native token-shard loader: mmap'd uint16 shards, per-rank disjoint spans, background prefetch into a pinned ring.
// Same slicing contract as the reference loaders (parameter-golf-rs/crates/pg-data/src/token_stream.rs:222-248,
// train_gpt.py:486-494): per micro-step every rank skips rank*(L+1) tokens, takes L+1, skips the other ranks' spans.
#pragma once
#include <stdint.h>

#include <condition_variable>
#include <mutex>
#include <string>
#include <thread>
#include <vector>

namespace pgb {

struct ShardMap {
  const uint16_t* tokens = nullptr;   // payload (after the 1024-byte header)
  long long count = 0;
  void* base = nullptr;
  size_t bytes = 0;
};

class ShardLoader {
 public:
  ShardLoader(std::vector<std::string> files, int rank, int world);
  ~ShardLoader();
  ShardLoader(const ShardLoader&) = delete;
  ShardLoader& operator=(const ShardLoader&) = delete;

  // Synchronous API (stream position is that of the calling thread; not to be mixed with a running prefetch).
  void take(uint16_t* out, long long n);
  void skip(long long n);
  void next_span(uint16_t* out, long long global_tokens, int grad_accum);   // writes global/(world*accum)+1 tokens
  int file_idx() const { return file_idx_; }
  long long pos() const { return pos_; }
  void restore(int file_idx, long long pos);

  // Prefetch: a worker thread runs ahead of the consumer in a ring of `depth` page-locked buffers (plain memory when
  // no CUDA device is usable).  next_prefetched() returns the oldest ready span; the `keep` most recently returned
  // spans are never overwritten, so a returned pointer stays valid for the next keep-1 calls (long enough for the
  // asynchronous host-to-device copies of one optimizer step when keep = grad_accum).  depth > keep.
  void start_prefetch(long long global_tokens, int grad_accum, int depth, int keep);
  const uint16_t* next_prefetched(int* file_idx_after, long long* pos_after);
  void stop_prefetch();
  long long span_tokens() const { return span_; }
  bool pinned() const { return pinned_; }

 private:
  void open(int idx);
  void worker();

  std::vector<std::string> files_;
  int rank_, world_;
  ShardMap cur_;
  int file_idx_ = 0;
  long long pos_ = 0;

  // prefetch state
  std::thread thread_;
  std::mutex mu_;
  std::condition_variable cv_;
  std::vector<uint16_t*> ring_;
  std::vector<int> ring_file_;
  std::vector<long long> ring_pos_;
  bool pinned_ = false;
  long long span_ = 0, global_ = 0;
  int accum_ = 1, keep_ = 1;
  long long produced_ = 0, consumed_ = 0;
  bool stop_ = false, running_ = false;
  std::string error_;
};

}  // namespace pgb
