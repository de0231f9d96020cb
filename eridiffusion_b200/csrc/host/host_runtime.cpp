// Native host runtime: memory-mapped safetensors access with pinned double-buffered host->device
// streaming, a size-classed pinned-memory pool, SHA-256, and the deterministic xorshift
// permutation used by the manifest loaders. Plain C ABI for ctypes.
//
// Reference counterparts: StrictMmapLoader / STFile (crates/common/weights/src/strict_loader.rs,
// crates/common/io/src/lib.rs:27-68, which stages through an f32 host Vec), pinned alloc + async
// memcpy (crates/core/cuda/utils_pinned.cu:4-20), PinnedPool / HostStager
// (crates/training/src/io.rs:16-190), manifest index hashing (flux/data_loader.rs:488-617).
#include <cuda_runtime.h>
#include <fcntl.h>
#include <stdint.h>
#include <string.h>
#include <sys/mman.h>
#include <sys/stat.h>
#include <unistd.h>

#include <map>
#include <mutex>
#include <string>
#include <vector>

namespace {

struct StFile {
  int fd = -1;
  uint8_t* base = nullptr;
  size_t size = 0;
  uint64_t header_len = 0;
  std::string header;
};

struct PinnedPool {
  std::mutex mu;
  std::map<size_t, std::vector<void*>> free_lists;   // size class -> buffers
  std::map<void*, size_t> owned;                     // ptr -> class
  std::map<void*, bool> is_pinned;
  size_t held = 0, hits = 0, misses = 0;
};
PinnedPool g_pool;

size_t size_class(size_t n) {
  size_t c = 4096;
  while (c < n) c <<= 1;
  return c;
}

// ------------------------------------------------------------------ SHA-256
struct Sha256 {
  uint32_t h[8];
  uint8_t buf[64];
  uint64_t len = 0;
  size_t fill = 0;
};
const uint32_t K256[64] = {
    0x428a2f98, 0x71374491, 0xb5c0fbcf, 0xe9b5dba5, 0x3956c25b, 0x59f111f1, 0x923f82a4, 0xab1c5ed5,
    0xd807aa98, 0x12835b01, 0x243185be, 0x550c7dc3, 0x72be5d74, 0x80deb1fe, 0x9bdc06a7, 0xc19bf174,
    0xe49b69c1, 0xefbe4786, 0x0fc19dc6, 0x240ca1cc, 0x2de92c6f, 0x4a7484aa, 0x5cb0a9dc, 0x76f988da,
    0x983e5152, 0xa831c66d, 0xb00327c8, 0xbf597fc7, 0xc6e00bf3, 0xd5a79147, 0x06ca6351, 0x14292967,
    0x27b70a85, 0x2e1b2138, 0x4d2c6dfc, 0x53380d13, 0x650a7354, 0x766a0abb, 0x81c2c92e, 0x92722c85,
    0xa2bfe8a1, 0xa81a664b, 0xc24b8b70, 0xc76c51a3, 0xd192e819, 0xd6990624, 0xf40e3585, 0x106aa070,
    0x19a4c116, 0x1e376c08, 0x2748774c, 0x34b0bcb5, 0x391c0cb3, 0x4ed8aa4a, 0x5b9cca4f, 0x682e6ff3,
    0x748f82ee, 0x78a5636f, 0x84c87814, 0x8cc70208, 0x90befffa, 0xa4506ceb, 0xbef9a3f7, 0xc67178f2};
inline uint32_t rotr(uint32_t x, int n) { return (x >> n) | (x << (32 - n)); }
void sha_block(Sha256& s, const uint8_t* p) {
  uint32_t w[64];
  for (int i = 0; i < 16; ++i)
    w[i] = (uint32_t)p[4 * i] << 24 | (uint32_t)p[4 * i + 1] << 16 | (uint32_t)p[4 * i + 2] << 8 | p[4 * i + 3];
  for (int i = 16; i < 64; ++i) {
    uint32_t s0 = rotr(w[i - 15], 7) ^ rotr(w[i - 15], 18) ^ (w[i - 15] >> 3);
    uint32_t s1 = rotr(w[i - 2], 17) ^ rotr(w[i - 2], 19) ^ (w[i - 2] >> 10);
    w[i] = w[i - 16] + s0 + w[i - 7] + s1;
  }
  uint32_t a = s.h[0], b = s.h[1], c = s.h[2], d = s.h[3], e = s.h[4], f = s.h[5], g = s.h[6], h = s.h[7];
  for (int i = 0; i < 64; ++i) {
    uint32_t S1 = rotr(e, 6) ^ rotr(e, 11) ^ rotr(e, 25), ch = (e & f) ^ (~e & g);
    uint32_t t1 = h + S1 + ch + K256[i] + w[i];
    uint32_t S0 = rotr(a, 2) ^ rotr(a, 13) ^ rotr(a, 22), mj = (a & b) ^ (a & c) ^ (b & c);
    uint32_t t2 = S0 + mj;
    h = g; g = f; f = e; e = d + t1; d = c; c = b; b = a; a = t1 + t2;
  }
  s.h[0] += a; s.h[1] += b; s.h[2] += c; s.h[3] += d; s.h[4] += e; s.h[5] += f; s.h[6] += g; s.h[7] += h;
}
void sha_init(Sha256& s) {
  const uint32_t iv[8] = {0x6a09e667, 0xbb67ae85, 0x3c6ef372, 0xa54ff53a, 0x510e527f, 0x9b05688c, 0x1f83d9ab, 0x5be0cd19};
  memcpy(s.h, iv, sizeof(iv));
  s.len = 0;
  s.fill = 0;
}
void sha_update(Sha256& s, const uint8_t* p, size_t n) {
  s.len += n;
  while (n) {
    size_t take = 64 - s.fill < n ? 64 - s.fill : n;
    memcpy(s.buf + s.fill, p, take);
    s.fill += take; p += take; n -= take;
    if (s.fill == 64) { sha_block(s, s.buf); s.fill = 0; }
  }
}
void sha_final(Sha256& s, uint8_t out[32]) {
  uint64_t bits = s.len * 8;
  uint8_t pad = 0x80;
  sha_update(s, &pad, 1);
  uint8_t z = 0;
  while (s.fill != 56) sha_update(s, &z, 1);
  uint8_t lb[8];
  for (int i = 0; i < 8; ++i) lb[i] = (uint8_t)(bits >> (56 - 8 * i));
  sha_update(s, lb, 8);
  for (int i = 0; i < 8; ++i) { out[4 * i] = s.h[i] >> 24; out[4 * i + 1] = s.h[i] >> 16; out[4 * i + 2] = s.h[i] >> 8; out[4 * i + 3] = s.h[i]; }
}

}  // namespace

extern "C" {

// ------------------------------------------------------------------ pinned pool
void* eri_pinned_alloc(long long nbytes) {
  size_t cls = size_class((size_t)nbytes);
  std::lock_guard<std::mutex> g(g_pool.mu);
  auto& fl = g_pool.free_lists[cls];
  if (!fl.empty()) {
    void* p = fl.back();
    fl.pop_back();
    g_pool.hits++;
    return p;
  }
  g_pool.misses++;
  void* p = nullptr;
  bool pinned = cudaHostAlloc(&p, cls, cudaHostAllocPortable) == cudaSuccess;
  if (!pinned) {
    cudaGetLastError();
    if (posix_memalign(&p, 4096, cls) != 0) return nullptr;   // no CUDA runtime: pageable fallback
  }
  g_pool.owned[p] = cls;
  g_pool.is_pinned[p] = pinned;
  g_pool.held += cls;
  return p;
}
void eri_pinned_free(void* p) {
  std::lock_guard<std::mutex> g(g_pool.mu);
  auto it = g_pool.owned.find(p);
  if (it != g_pool.owned.end()) g_pool.free_lists[it->second].push_back(p);
}
void eri_pinned_trim() {
  std::lock_guard<std::mutex> g(g_pool.mu);
  for (auto& kv : g_pool.free_lists)
    for (void* p : kv.second) {
      if (g_pool.is_pinned[p]) cudaFreeHost(p); else free(p);
      g_pool.held -= g_pool.owned[p];
      g_pool.owned.erase(p);
      g_pool.is_pinned.erase(p);
    }
  g_pool.free_lists.clear();
}
void eri_pinned_stats(long long* held, long long* hits, long long* misses) {
  std::lock_guard<std::mutex> g(g_pool.mu);
  *held = (long long)g_pool.held; *hits = (long long)g_pool.hits; *misses = (long long)g_pool.misses;
}

// ------------------------------------------------------------------ safetensors mmap
void* eri_st_open(const char* path) {
  StFile* f = new StFile();
  f->fd = open(path, O_RDONLY);
  if (f->fd < 0) { delete f; return nullptr; }
  struct stat sb;
  if (fstat(f->fd, &sb) != 0 || sb.st_size < 8) { close(f->fd); delete f; return nullptr; }
  f->size = (size_t)sb.st_size;
  f->base = (uint8_t*)mmap(nullptr, f->size, PROT_READ, MAP_PRIVATE, f->fd, 0);
  if (f->base == MAP_FAILED) { close(f->fd); delete f; return nullptr; }
  memcpy(&f->header_len, f->base, 8);
  if (f->header_len > f->size - 8 || f->header_len > (100ull << 20)) {
    munmap(f->base, f->size); close(f->fd); delete f; return nullptr;
  }
  f->header.assign((const char*)f->base + 8, (size_t)f->header_len);
  return f;
}
const char* eri_st_header(void* h) { return ((StFile*)h)->header.c_str(); }
long long eri_st_data_offset(void* h) { return 8 + (long long)((StFile*)h)->header_len; }
long long eri_st_size(void* h) { return (long long)((StFile*)h)->size; }
const void* eri_st_data(void* h) { StFile* f = (StFile*)h; return f->base + 8 + f->header_len; }
void eri_st_close(void* h) {
  StFile* f = (StFile*)h;
  if (!f) return;
  munmap(f->base, f->size);
  close(f->fd);
  delete f;
}
// Copy `nbytes` at payload offset `off` to host memory.
int eri_st_read_host(void* h, long long off, long long nbytes, void* dst) {
  StFile* f = (StFile*)h;
  if (8 + f->header_len + off + nbytes > f->size) return -1;
  memcpy(dst, f->base + 8 + f->header_len + off, (size_t)nbytes);
  return 0;
}
// Stream `nbytes` at payload offset `off` to device memory through two pinned staging buffers:
// the memcpy of chunk i+1 from the page cache overlaps the DMA of chunk i.
int eri_st_read_device(void* h, long long off, long long nbytes, void* dst_dev, void* stream) {
  StFile* f = (StFile*)h;
  if (8 + f->header_len + off + nbytes > f->size) return -1;
  const size_t chunk = 16u << 20;
  void* stage[2] = {eri_pinned_alloc(chunk), eri_pinned_alloc(chunk)};
  cudaEvent_t ev[2];
  cudaEventCreateWithFlags(&ev[0], cudaEventDisableTiming);
  cudaEventCreateWithFlags(&ev[1], cudaEventDisableTiming);
  const uint8_t* src = f->base + 8 + f->header_len + off;
  int rc = 0, i = 0;
  for (size_t done = 0; done < (size_t)nbytes; done += chunk, ++i) {
    int b = i & 1;
    size_t n = (size_t)nbytes - done < chunk ? (size_t)nbytes - done : chunk;
    if (i >= 2) cudaEventSynchronize(ev[b]);
    memcpy(stage[b], src + done, n);
    if (cudaMemcpyAsync((uint8_t*)dst_dev + done, stage[b], n, cudaMemcpyHostToDevice, (cudaStream_t)stream) != cudaSuccess) { rc = -2; break; }
    cudaEventRecord(ev[b], (cudaStream_t)stream);
  }
  cudaEventSynchronize(ev[0]);
  cudaEventSynchronize(ev[1]);
  cudaEventDestroy(ev[0]);
  cudaEventDestroy(ev[1]);
  eri_pinned_free(stage[0]);
  eri_pinned_free(stage[1]);
  return rc;
}
// Write a safetensors file: header JSON (already padded by the caller) + tensors in order.
int eri_st_write(const char* path, const char* header, long long header_len, int n, const void** ptrs, const long long* sizes) {
  std::string tmp = std::string(path) + ".tmp";
  int fd = open(tmp.c_str(), O_WRONLY | O_CREAT | O_TRUNC, 0644);
  if (fd < 0) return -1;
  uint64_t hl = (uint64_t)header_len;
  bool ok = write(fd, &hl, 8) == 8 && write(fd, header, (size_t)header_len) == (ssize_t)header_len;
  for (int i = 0; ok && i < n; ++i) {
    size_t left = (size_t)sizes[i];
    const uint8_t* p = (const uint8_t*)ptrs[i];
    while (left) {
      ssize_t w = write(fd, p, left);
      if (w <= 0) { ok = false; break; }
      left -= (size_t)w; p += w;
    }
  }
  close(fd);
  if (!ok) { unlink(tmp.c_str()); return -2; }
  return rename(tmp.c_str(), path);
}

// ------------------------------------------------------------------ hashing / shuffling
int eri_sha256_file(const char* path, char out_hex[65]) {
  int fd = open(path, O_RDONLY);
  if (fd < 0) return -1;
  Sha256 s;
  sha_init(s);
  std::vector<uint8_t> buf(1 << 20);
  ssize_t n;
  while ((n = read(fd, buf.data(), buf.size())) > 0) sha_update(s, buf.data(), (size_t)n);
  close(fd);
  uint8_t d[32];
  sha_final(s, d);
  static const char* hx = "0123456789abcdef";
  for (int i = 0; i < 32; ++i) { out_hex[2 * i] = hx[d[i] >> 4]; out_hex[2 * i + 1] = hx[d[i] & 15]; }
  out_hex[64] = 0;
  return 0;
}
int eri_sha256_bytes(const void* p, long long n, char out_hex[65]) {
  Sha256 s;
  sha_init(s);
  sha_update(s, (const uint8_t*)p, (size_t)n);
  uint8_t d[32];
  sha_final(s, d);
  static const char* hx = "0123456789abcdef";
  for (int i = 0; i < 32; ++i) { out_hex[2 * i] = hx[d[i] >> 4]; out_hex[2 * i + 1] = hx[d[i] & 15]; }
  out_hex[64] = 0;
  return 0;
}
// Same sequence as data.xorshift_permutation (Fisher-Yates driven by xorshift64*).
void eri_xorshift_permutation(long long n, unsigned long long seed, long long* out) {
  unsigned long long s = seed * 0x9E3779B97F4A7C15ull + 0xD1B54A32D192ED03ull;
  if (!s) s = 0x2545F4914F6CDD1Dull;
  for (long long i = 0; i < n; ++i) out[i] = i;
  for (long long i = n - 1; i > 0; --i) {
    s ^= s >> 12; s ^= s << 25; s ^= s >> 27;
    unsigned long long r = s * 0x2545F4914F6CDD1Dull;
    long long j = (long long)(r % (unsigned long long)(i + 1));
    long long t = out[i]; out[i] = out[j]; out[j] = t;
  }
}

}  // extern "C"
