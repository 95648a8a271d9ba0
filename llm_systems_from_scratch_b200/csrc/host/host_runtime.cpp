// Host-side runtime pieces that sit on the per-step path of the loader and the serving scheduler, as a plain
// C ABI (loaded with ctypes, no Python objects cross the boundary):
//
//   b200h_gather_windows   random-window batch assembly (the reference's sample_batch, llm-core/llm_core/
//                          dataloader.py:8-27, builds the same windows with numpy fancy indexing): copies
//                          batch windows of a uint32 token array (usually an mmap) into a pinned int64 staging
//                          buffer, widening on the fly, split over worker threads for large batches
//   b200h_pages_*          LIFO free-list page allocator of the paged KV cache with O(1) take / give per page
//   b200h_slots            flat cache slots (page * page_size + offset) of a token range of one request
//   b200h_block_table      padded int32 block-table rows for a batch of requests
#include <cstdint>
#include <cstring>
#include <thread>
#include <vector>

namespace {

struct PagePool {
  std::vector<int32_t> free_list;   // back = next page handed out
  int32_t num_pages;
};

void gather_range(const uint32_t* tokens, const int64_t* starts, int width, int64_t* out, int b0, int b1) {
  for (int b = b0; b < b1; ++b) {
    const uint32_t* src = tokens + starts[b];
    int64_t* dst = out + (int64_t)b * width;
    for (int j = 0; j < width; ++j) dst[j] = (int64_t)src[j];
  }
}

}  // namespace

extern "C" {

// out[b][j] = tokens[starts[b] + j] for j < width.  The caller guarantees starts[b] + width <= n_tokens.
int b200h_gather_windows(const uint32_t* tokens, long long n_tokens, const int64_t* starts, int batch, int width,
                         int64_t* out, int threads) {
  if (batch < 0 || width <= 0) return -1;
  for (int b = 0; b < batch; ++b)
    if (starts[b] < 0 || starts[b] + width > n_tokens) return -2;
  const long long work = (long long)batch * width;
  if (threads <= 1 || work < (1 << 16) || batch < 2) {
    gather_range(tokens, starts, width, out, 0, batch);
    return 0;
  }
  if (threads > batch) threads = batch;
  std::vector<std::thread> pool;
  pool.reserve(threads);
  for (int t = 0; t < threads; ++t) {
    const int b0 = (int)((long long)batch * t / threads), b1 = (int)((long long)batch * (t + 1) / threads);
    pool.emplace_back(gather_range, tokens, starts, width, out, b0, b1);
  }
  for (auto& th : pool) th.join();
  return 0;
}

void* b200h_pages_create(int num_pages) {
  if (num_pages < 0) return nullptr;
  auto* p = new PagePool;
  p->num_pages = num_pages;
  p->free_list.resize(num_pages);
  for (int i = 0; i < num_pages; ++i) p->free_list[i] = num_pages - 1 - i;   // page 0 is handed out first
  return p;
}

void b200h_pages_destroy(void* h) { delete static_cast<PagePool*>(h); }

int b200h_pages_free(void* h) { return (int)static_cast<PagePool*>(h)->free_list.size(); }

// Takes n pages (LIFO); 0 on success, -1 when fewer than n are free (nothing is taken then).
int b200h_pages_take(void* h, int n, int32_t* out) {
  auto* p = static_cast<PagePool*>(h);
  if (n < 0 || (size_t)n > p->free_list.size()) return -1;
  for (int i = 0; i < n; ++i) {
    out[i] = p->free_list.back();
    p->free_list.pop_back();
  }
  return 0;
}

// Returns pages to the pool so that the first page of `pages` is the next one handed out.
int b200h_pages_give(void* h, const int32_t* pages, int n) {
  auto* p = static_cast<PagePool*>(h);
  for (int i = 0; i < n; ++i)
    if (pages[i] < 0 || pages[i] >= p->num_pages) return -1;
  for (int i = n - 1; i >= 0; --i) p->free_list.push_back(pages[i]);
  return 0;
}

// out[i] = pages[(start + i) / page_size] * page_size + (start + i) % page_size
int b200h_slots(const int32_t* pages, int n_pages, int page_size, int start, int count, int64_t* out) {
  if (page_size <= 0 || start < 0 || count < 0 || (long long)start + count > (long long)n_pages * page_size) return -1;
  for (int i = 0; i < count; ++i) {
    const int t = start + i;
    out[i] = (int64_t)pages[t / page_size] * page_size + t % page_size;
  }
  return 0;
}

// Row r of `table` (rows x width, int32) = the page ids of request r, padded with `pad`.  `pages` holds the
// requests' page lists back to back, `offsets` (rows + 1) their boundaries.
int b200h_block_table(const int32_t* pages, const int32_t* offsets, int rows, int width, int32_t pad, int32_t* table) {
  for (int r = 0; r < rows; ++r) {
    const int n = offsets[r + 1] - offsets[r];
    if (n < 0 || n > width) return -1;
    int32_t* row = table + (long long)r * width;
    std::memcpy(row, pages + offsets[r], sizeof(int32_t) * n);
    for (int j = n; j < width; ++j) row[j] = pad;
  }
  return 0;
}

}  // extern "C"
