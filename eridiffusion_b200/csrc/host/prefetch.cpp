// Native read-ahead for the cached-embedding loaders and for block streaming: worker threads read
// byte ranges of files (safetensors payloads) into buffers from the pinned pool ahead of the
// training loop, so that the step only sees a finished host buffer it can copy to the device
// asynchronously.
//
//   h = eri_prefetch_create(threads, max_inflight)
//   t = eri_prefetch_submit(h, path, offset, nbytes)      // returns a ticket >= 0, never blocks on IO
//   eri_prefetch_wait(h, t, &ptr, &nbytes)                // blocks until that range is in memory
//   eri_prefetch_release(h, t)                            // buffer goes back to the pinned pool
//   eri_prefetch_destroy(h)
//
// submit blocks (back-pressure) while max_inflight tickets are outstanding. Errors (missing file,
// short read) are reported by wait as a negative code; the ticket must still be released.
//
// Reference counterparts: the manifest loaders read and stage every sample synchronously inside
// next_batch (crates/training/src/flux/data_loader.rs:641-656, sdxl/data_loader.rs:364-374);
// BlockSwapManager::prefetch_next is declared with an empty async prefetch file
// (crates/common/blockswap/src/prefetch.rs:1).
#include <fcntl.h>
#include <stdint.h>
#include <sys/stat.h>
#include <unistd.h>

#include <condition_variable>
#include <deque>
#include <map>
#include <mutex>
#include <string>
#include <thread>
#include <vector>

extern "C" void* eri_pinned_alloc(long long nbytes);
extern "C" void eri_pinned_free(void* p);

namespace {

struct Job {
  long long ticket;
  std::string path;
  long long offset, nbytes;
};

struct Slot {
  void* ptr = nullptr;
  long long nbytes = 0;
  int status = 1;   // 1 pending, 0 done, < 0 error
};

struct Prefetcher {
  std::mutex mu;
  std::condition_variable cv_work, cv_done, cv_room;
  std::deque<Job> queue;
  std::map<long long, Slot> slots;
  std::vector<std::thread> workers;
  long long next_ticket = 0;
  int max_inflight = 8;
  bool stop = false;
  long long bytes_read = 0;
};

int read_range(const std::string& path, long long offset, long long nbytes, void* dst) {
  int fd = open(path.c_str(), O_RDONLY);
  if (fd < 0) return -2;
  long long done = 0;
  while (done < nbytes) {
    ssize_t r = pread(fd, (char*)dst + done, (size_t)(nbytes - done), (off_t)(offset + done));
    if (r <= 0) {
      close(fd);
      return -3;   // short read / IO error
    }
    done += r;
  }
  close(fd);
  return 0;
}

void worker(Prefetcher* p) {
  for (;;) {
    Job job;
    {
      std::unique_lock<std::mutex> lk(p->mu);
      p->cv_work.wait(lk, [&] { return p->stop || !p->queue.empty(); });
      if (p->stop && p->queue.empty()) return;
      job = p->queue.front();
      p->queue.pop_front();
    }
    void* buf = eri_pinned_alloc(job.nbytes > 0 ? job.nbytes : 1);
    int st = buf ? read_range(job.path, job.offset, job.nbytes, buf) : -4;
    {
      std::lock_guard<std::mutex> lk(p->mu);
      Slot& s = p->slots[job.ticket];
      s.ptr = buf;
      s.nbytes = job.nbytes;
      s.status = st;
      if (st == 0) p->bytes_read += job.nbytes;
    }
    p->cv_done.notify_all();
  }
}

}  // namespace

extern "C" {

void* eri_prefetch_create(int threads, int max_inflight) {
  Prefetcher* p = new Prefetcher();
  p->max_inflight = max_inflight > 0 ? max_inflight : 8;
  if (threads < 1) threads = 1;
  for (int i = 0; i < threads; ++i) p->workers.emplace_back(worker, p);
  return p;
}

long long eri_prefetch_submit(void* h, const char* path, long long offset, long long nbytes) {
  Prefetcher* p = (Prefetcher*)h;
  if (!p || !path || offset < 0 || nbytes < 0) return -1;
  std::unique_lock<std::mutex> lk(p->mu);
  p->cv_room.wait(lk, [&] { return p->stop || (int)p->slots.size() < p->max_inflight; });
  if (p->stop) return -1;
  const long long t = p->next_ticket++;
  p->slots[t] = Slot();
  p->queue.push_back(Job{t, path, offset, nbytes});
  lk.unlock();
  p->cv_work.notify_one();
  return t;
}

// Returns 0 and the buffer, or a negative code: -1 unknown ticket, -2 cannot open, -3 short read,
// -4 out of memory.
int eri_prefetch_wait(void* h, long long ticket, void** ptr, long long* nbytes) {
  Prefetcher* p = (Prefetcher*)h;
  std::unique_lock<std::mutex> lk(p->mu);
  auto it = p->slots.find(ticket);
  if (it == p->slots.end()) return -1;
  p->cv_done.wait(lk, [&] { return p->slots[ticket].status != 1; });
  const Slot& s = p->slots[ticket];
  if (ptr) *ptr = s.ptr;
  if (nbytes) *nbytes = s.nbytes;
  return s.status;
}

int eri_prefetch_release(void* h, long long ticket) {
  Prefetcher* p = (Prefetcher*)h;
  void* buf = nullptr;
  {
    std::unique_lock<std::mutex> lk(p->mu);
    auto it = p->slots.find(ticket);
    if (it == p->slots.end()) return -1;
    p->cv_done.wait(lk, [&] { return p->slots[ticket].status != 1; });   // never free under a reader
    buf = p->slots[ticket].ptr;
    p->slots.erase(ticket);
  }
  if (buf) eri_pinned_free(buf);
  p->cv_room.notify_one();
  return 0;
}

long long eri_prefetch_bytes_read(void* h) {
  Prefetcher* p = (Prefetcher*)h;
  std::lock_guard<std::mutex> lk(p->mu);
  return p->bytes_read;
}

void eri_prefetch_destroy(void* h) {
  Prefetcher* p = (Prefetcher*)h;
  if (!p) return;
  {
    std::lock_guard<std::mutex> lk(p->mu);
    p->stop = true;
    p->queue.clear();
  }
  p->cv_work.notify_all();
  p->cv_room.notify_all();
  for (auto& t : p->workers) t.join();
  for (auto& kv : p->slots)
    if (kv.second.ptr) eri_pinned_free(kv.second.ptr);
  delete p;
}

}  // extern "C"
