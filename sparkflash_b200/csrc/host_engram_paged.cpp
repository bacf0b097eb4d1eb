// Engram tables that stay on storage: a paged reader over a packed table file with an LRU page cache and a read-ahead
// thread.
//
// The two Engram tables are ~190 GiB of FP8 rows.  Where they do not fit beside the model (one or two GPUs), the packed
// file stays on NVMe and a step reads only the rows its tokens hash to: 24 rows per token and layer, 272 bytes each.
// Rows are read in pages (a page = `page_rows` consecutive rows, one pread); pages are cached with least-recently-used
// eviction; and because the n-gram ids of the next positions are known as soon as the tokens are (a prompt's whole id
// list at admission, a draft block's ids before it is verified), the serving loop asks for them ahead of time and a
// background thread pulls the pages in while the GPU runs the current step.
//
// Thread-safety: one mutex guards the cache; a page being loaded is marked so that a demand read of the same page waits
// for it instead of reading it twice.
//
// Reference behaviour: crates/sparkflash-engram/src/{packer,paged,store}.rs (packed NVMe file, paged reader, prefetch,
// cache), crates/sparkflash-deepseek-forward/src/tp4_forward/spec.rs:134-265,934-945 (io_uring gather, read-ahead of the
// next positions' rows).
#include <fcntl.h>
#include <stdint.h>
#include <string.h>
#include <sys/stat.h>
#include <unistd.h>

#include <condition_variable>
#include <deque>
#include <list>
#include <mutex>
#include <thread>
#include <unordered_map>
#include <vector>

namespace {

struct Page {
  int64_t id = -1;
  std::vector<uint8_t> data;
  bool ready = false;
  std::list<int64_t>::iterator lru;
};

struct Paged {
  int fd = -1;
  int64_t rows = 0;
  int stride = 0, page_rows = 0, capacity = 0;
  std::mutex mu;
  std::condition_variable cv_ready, cv_work;
  std::unordered_map<int64_t, Page*> pages;
  std::list<int64_t> lru;            // front = most recent
  std::deque<int64_t> queue;         // pages requested ahead of time
  std::thread worker;
  bool stop = false;
  uint64_t hits = 0, misses = 0, prefetched = 0, evictions = 0, bytes_read = 0, waits = 0;
};

// page lookup with the lock held; returns the page (maybe not ready) or null
Page* find(Paged* p, int64_t id) {
  auto it = p->pages.find(id);
  return it == p->pages.end() ? nullptr : it->second;
}

void touch(Paged* p, Page* pg) {
  p->lru.erase(pg->lru);
  p->lru.push_front(pg->id);
  pg->lru = p->lru.begin();
}

// make room and insert an empty (not ready) page; lock held.  Never evicts a page that is still loading.
Page* insert(Paged* p, int64_t id) {
  while ((int)p->pages.size() >= p->capacity) {
    bool evicted = false;
    for (auto it = p->lru.rbegin(); it != p->lru.rend(); ++it) {
      Page* v = p->pages[*it];
      if (!v->ready) continue;
      p->lru.erase(v->lru);
      p->pages.erase(v->id);
      delete v;
      ++p->evictions;
      evicted = true;
      break;
    }
    if (!evicted) break;     // everything resident is in flight: run over capacity for a moment rather than deadlock
  }
  Page* pg = new Page();
  pg->id = id;
  pg->data.resize((size_t)p->page_rows * p->stride);
  p->lru.push_front(id);
  pg->lru = p->lru.begin();
  p->pages[id] = pg;
  return pg;
}

// read the page's bytes without the lock; rows past the table's end read as zeros
bool load(Paged* p, Page* pg) {
  const int64_t first = pg->id * p->page_rows;
  int64_t want = p->page_rows;
  if (first + want > p->rows) want = p->rows - first;
  memset(pg->data.data(), 0, pg->data.size());
  size_t done = 0;
  const size_t total = want > 0 ? (size_t)want * p->stride : 0;
  while (done < total) {
    const ssize_t r = pread(p->fd, pg->data.data() + done, total - done, (off_t)((size_t)first * p->stride + done));
    if (r <= 0) return false;
    done += (size_t)r;
  }
  return true;
}

void worker_loop(Paged* p) {
  std::unique_lock<std::mutex> lk(p->mu);
  for (;;) {
    p->cv_work.wait(lk, [&] { return p->stop || !p->queue.empty(); });
    if (p->stop) return;
    const int64_t id = p->queue.front();
    p->queue.pop_front();
    if (find(p, id)) continue;
    Page* pg = insert(p, id);
    lk.unlock();
    const bool ok = load(p, pg);
    lk.lock();
    p->bytes_read += pg->data.size();
    ++p->prefetched;
    pg->ready = true;       // a failed read leaves zeros: the demand path re-reads and reports the error
    if (!ok) { p->lru.erase(pg->lru); p->pages.erase(pg->id); delete pg; }
    p->cv_ready.notify_all();
  }
}

}  // namespace

extern "C" {

void* sfb_epaged_open(const char* path, int64_t rows, int stride, int page_rows, int cache_pages) {
  if (rows < 0 || stride <= 0 || page_rows <= 0 || cache_pages <= 0) return nullptr;
  const int fd = open(path, O_RDONLY);
  if (fd < 0) return nullptr;
  struct stat st;
  if (fstat(fd, &st) || (int64_t)st.st_size < rows * (int64_t)stride) { close(fd); return nullptr; }
  Paged* p = new Paged();
  p->fd = fd; p->rows = rows; p->stride = stride; p->page_rows = page_rows; p->capacity = cache_pages;
  p->worker = std::thread(worker_loop, p);
  return p;
}

void sfb_epaged_close(void* h) {
  Paged* p = (Paged*)h;
  {
    std::lock_guard<std::mutex> lk(p->mu);
    p->stop = true;
  }
  p->cv_work.notify_all();
  if (p->worker.joinable()) p->worker.join();
  for (auto& kv : p->pages) delete kv.second;
  close(p->fd);
  delete p;
}

// Copy the rows `ids[0..n)` into out (n x stride bytes).  Ids outside [0, rows) give zero rows.  Returns 0, or 1 when a
// read failed.
int sfb_epaged_gather(void* h, const int64_t* ids, int n, uint8_t* out) {
  Paged* p = (Paged*)h;
  for (int i = 0; i < n; ++i) {
    uint8_t* dst = out + (size_t)i * p->stride;
    const int64_t id = ids[i];
    if (id < 0 || id >= p->rows) { memset(dst, 0, p->stride); continue; }
    const int64_t pid = id / p->page_rows;
    std::unique_lock<std::mutex> lk(p->mu);
    Page* pg = find(p, pid);
    if (pg) {
      if (!pg->ready) {
        ++p->waits;
        p->cv_ready.wait(lk, [&] { Page* q = find(p, pid); return q == nullptr || q->ready; });
        pg = find(p, pid);
      }
      if (pg) { ++p->hits; touch(p, pg); }
    }
    if (!pg) {
      ++p->misses;
      pg = insert(p, pid);
      lk.unlock();
      const bool ok = load(p, pg);
      lk.lock();
      p->bytes_read += pg->data.size();
      pg->ready = true;
      p->cv_ready.notify_all();
      if (!ok) { p->lru.erase(pg->lru); p->pages.erase(pid); delete pg; memset(dst, 0, p->stride); return 1; }
    }
    memcpy(dst, pg->data.data() + (size_t)(id - pid * p->page_rows) * p->stride, p->stride);
  }
  return 0;
}

// Ask for the pages of these rows ahead of time; returns the number of pages queued.
int sfb_epaged_prefetch(void* h, const int64_t* ids, int n) {
  Paged* p = (Paged*)h;
  int queued = 0;
  {
    std::lock_guard<std::mutex> lk(p->mu);
    for (int i = 0; i < n; ++i) {
      if (ids[i] < 0 || ids[i] >= p->rows) continue;
      const int64_t pid = ids[i] / p->page_rows;
      if (find(p, pid)) continue;
      bool dup = false;
      for (int64_t q : p->queue) if (q == pid) { dup = true; break; }
      if (dup) continue;
      p->queue.push_back(pid);
      ++queued;
    }
  }
  if (queued) p->cv_work.notify_all();
  return queued;
}

// Block until the read-ahead queue is empty and nothing is loading (tests, orderly shutdown).
void sfb_epaged_drain(void* h) {
  Paged* p = (Paged*)h;
  std::unique_lock<std::mutex> lk(p->mu);
  p->cv_ready.wait(lk, [&] {
    if (!p->queue.empty()) return false;
    for (auto& kv : p->pages) if (!kv.second->ready) return false;
    return true;
  });
}

// out[0..7] = hits, misses, prefetched pages, evictions, bytes read, resident pages, waits on a loading page, queue length
void sfb_epaged_stats(void* h, uint64_t* out) {
  Paged* p = (Paged*)h;
  std::lock_guard<std::mutex> lk(p->mu);
  out[0] = p->hits; out[1] = p->misses; out[2] = p->prefetched; out[3] = p->evictions; out[4] = p->bytes_read;
  out[5] = p->pages.size(); out[6] = p->waits; out[7] = p->queue.size();
}

}  // extern "C"
