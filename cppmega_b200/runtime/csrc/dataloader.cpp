// Native token-stream reader and batch prefetcher.
//
// Reads the indexed dataset format the reference feeds to Megatron (`<prefix>.bin` = concatenated token ids,
// `<prefix>.idx` = header + per-document sizes / offsets; produced by its data pipeline,
// scripts/data_prep_parquet_to_megatron.py) and also a headerless raw token file.  Documents are concatenated
// into one stream; a sample is `seq_len + 1` consecutive tokens.  Sample order is a seeded permutation that is
// identical on every rank; rank r of n takes samples r, r+n, ...  A background thread fills a ring of
// pinned-host batches so the training loop never waits on the page cache.
#include <atomic>
#include <condition_variable>
#include <cstdint>
#include <cstdio>
#include <cstring>
#include <fcntl.h>
#include <mutex>
#include <random>
#include <string>
#include <sys/mman.h>
#include <sys/stat.h>
#include <thread>
#include <unistd.h>
#include <vector>

namespace {

struct Loader {
  int fd = -1;
  const uint8_t* base = nullptr;
  size_t bytes = 0;
  int token_bytes = 4;
  uint64_t num_tokens = 0;
  int seq_len = 0, micro_batch = 0, rank = 0, world = 1;
  uint64_t seed = 0, num_samples = 0;
  std::vector<uint64_t> order;
  uint64_t cursor = 0, epoch = 0;
  // ring
  int depth = 4;
  std::vector<int64_t*> slots;
  std::vector<int> state;           // 0 empty, 1 full
  int head = 0, tail = 0;
  std::mutex mu;
  std::condition_variable cv;
  std::thread worker;
  std::atomic<bool> stop{false};
  bool external_slots = false;
};

void reshuffle(Loader* L) {
  L->order.resize(L->num_samples);
  for (uint64_t i = 0; i < L->num_samples; ++i) L->order[i] = i;
  std::mt19937_64 gen(L->seed + 0x9E3779B97F4A7C15ull * (L->epoch + 1));
  for (uint64_t i = L->num_samples; i > 1; --i) {
    uint64_t j = gen() % i;
    std::swap(L->order[i - 1], L->order[j]);
  }
}

inline int64_t token_at(const Loader* L, uint64_t i) {
  switch (L->token_bytes) {
    case 2: return reinterpret_cast<const uint16_t*>(L->base)[i];
    case 4: return reinterpret_cast<const int32_t*>(L->base)[i];
    default: return reinterpret_cast<const int64_t*>(L->base)[i];
  }
}

void fill(Loader* L, int64_t* dst) {
  const int width = L->seq_len + 1;
  for (int b = 0; b < L->micro_batch; ++b) {
    uint64_t global = L->cursor * L->world + L->rank;
    if (global >= L->num_samples) {
      L->epoch++;
      reshuffle(L);
      L->cursor = 0;
      global = L->rank;
    }
    const uint64_t sample = L->order[global % L->num_samples];
    const uint64_t start = sample * (uint64_t)L->seq_len;
    for (int t = 0; t < width; ++t) dst[(size_t)b * width + t] = token_at(L, start + t);
    L->cursor++;
  }
}

void run(Loader* L) {
  while (!L->stop.load()) {
    std::unique_lock<std::mutex> lk(L->mu);
    L->cv.wait(lk, [&] { return L->stop.load() || L->state[L->head] == 0; });
    if (L->stop.load()) return;
    const int s = L->head;
    lk.unlock();
    fill(L, L->slots[s]);
    lk.lock();
    L->state[s] = 1;
    L->head = (L->head + 1) % L->depth;
    lk.unlock();
    L->cv.notify_all();
  }
}

}  // namespace

extern "C" {

// token_bytes: 2, 4 or 8.  header_bytes: bytes to skip at the start of the .bin (0 for Megatron .bin files).
void* cm_loader_open(const char* bin_path, int token_bytes, long long header_bytes, int seq_len, int micro_batch, int rank,
                     int world, unsigned long long seed, int depth) {
  Loader* L = new Loader();
  L->fd = ::open(bin_path, O_RDONLY);
  if (L->fd < 0) { delete L; return nullptr; }
  struct stat st;
  if (fstat(L->fd, &st) != 0 || st.st_size <= header_bytes) { ::close(L->fd); delete L; return nullptr; }
  L->bytes = (size_t)st.st_size;
  void* m = mmap(nullptr, L->bytes, PROT_READ, MAP_SHARED, L->fd, 0);
  if (m == MAP_FAILED) { ::close(L->fd); delete L; return nullptr; }
  madvise(m, L->bytes, MADV_RANDOM);
  L->base = reinterpret_cast<const uint8_t*>(m) + header_bytes;
  L->token_bytes = token_bytes;
  L->num_tokens = (L->bytes - header_bytes) / token_bytes;
  L->seq_len = seq_len; L->micro_batch = micro_batch; L->rank = rank; L->world = world; L->seed = seed;
  if (L->num_tokens < (uint64_t)seq_len + 1) { munmap(m, L->bytes); ::close(L->fd); delete L; return nullptr; }
  L->num_samples = (L->num_tokens - 1) / seq_len;
  L->depth = depth > 1 ? depth : 2;
  reshuffle(L);
  return L;
}

long long cm_loader_num_samples(void* h) { return (long long)static_cast<Loader*>(h)->num_samples; }
long long cm_loader_num_tokens(void* h) { return (long long)static_cast<Loader*>(h)->num_tokens; }

// Give the loader `depth` caller-owned buffers of micro_batch * (seq_len + 1) int64 each (e.g. pinned memory)
// and start the prefetch thread.
int cm_loader_start(void* h, int64_t* const* buffers, int n) {
  Loader* L = static_cast<Loader*>(h);
  if (n != L->depth) return -1;
  L->slots.assign(buffers, buffers + n);
  L->state.assign(n, 0);
  L->external_slots = true;
  L->worker = std::thread(run, L);
  return 0;
}

// Blocks until the next batch is ready; returns its slot index.  The slot stays valid until cm_loader_release.
int cm_loader_next(void* h) {
  Loader* L = static_cast<Loader*>(h);
  std::unique_lock<std::mutex> lk(L->mu);
  L->cv.wait(lk, [&] { return L->state[L->tail] == 1; });
  return L->tail;
}

void cm_loader_release(void* h) {
  Loader* L = static_cast<Loader*>(h);
  {
    std::lock_guard<std::mutex> lk(L->mu);
    L->state[L->tail] = 0;
    L->tail = (L->tail + 1) % L->depth;
  }
  L->cv.notify_all();
}

// Resume support: position expressed in batches consumed by this rank.
void cm_loader_state(void* h, unsigned long long* epoch, unsigned long long* cursor) {
  Loader* L = static_cast<Loader*>(h);
  *epoch = L->epoch;
  *cursor = L->cursor;
}

void cm_loader_close(void* h) {
  Loader* L = static_cast<Loader*>(h);
  L->stop.store(true);
  L->cv.notify_all();
  if (L->worker.joinable()) L->worker.join();
  // the mapping is released with the process; the loader keeps only a pointer past the header
  if (L->fd >= 0) ::close(L->fd);
  delete L;
}

}  // extern "C"
