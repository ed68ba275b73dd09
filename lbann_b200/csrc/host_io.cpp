// Host runtime (no CUDA): tensor container files for checkpoints and a small thread
// pool for mini-batch collation.
//
// Container format ("LBT1"): 16-byte file header {magic "LBT1", u32 version, u64 count
// (patched on close)} followed by one record per tensor:
//   u32 name_len, name bytes, u32 dtype, u32 ndim, u64 dims[ndim], u64 nbytes,
//   u32 crc32(data), data bytes (64-byte aligned start).
// The checkpoint layer (lbann_b200/io/checkpoint.py) stores model.bin / trainer.bin /
// *_ctx.bin / rng_state files in this format inside the reference's directory layout
// (src/callbacks/checkpoint.cpp:689-727).  Large payloads are written with several
// threads using pwrite.
#include <cstdint>
#include <cstdio>
#include <cstring>
#include <fcntl.h>
#include <string>
#include <sys/stat.h>
#include <thread>
#include <unistd.h>
#include <vector>

namespace {

uint32_t crc_table[256];
bool crc_ready = false;
void crc_init() {
  if (crc_ready) return;
  for (uint32_t i = 0; i < 256; ++i) {
    uint32_t c = i;
    for (int k = 0; k < 8; ++k) c = (c & 1) ? (0xEDB88320u ^ (c >> 1)) : (c >> 1);
    crc_table[i] = c;
  }
  crc_ready = true;
}
uint32_t crc32(const uint8_t* p, size_t n) {
  crc_init();
  uint32_t c = 0xFFFFFFFFu;
  for (size_t i = 0; i < n; ++i) c = crc_table[(c ^ p[i]) & 0xFF] ^ (c >> 8);
  return c ^ 0xFFFFFFFFu;
}

struct Entry {
  std::string name;
  uint32_t dtype = 0, ndim = 0, crc = 0;
  uint64_t dims[8] = {0};
  uint64_t nbytes = 0, offset = 0;
};

struct Writer {
  int fd = -1;
  uint64_t pos = 0, count = 0;
};
struct Reader {
  int fd = -1;
  std::vector<Entry> entries;
};

bool write_all(int fd, const void* buf, size_t n, uint64_t off) {
  const uint8_t* p = static_cast<const uint8_t*>(buf);
  while (n > 0) {
    ssize_t w = pwrite(fd, p, n, (off_t)off);
    if (w <= 0) return false;
    p += w; n -= (size_t)w; off += (uint64_t)w;
  }
  return true;
}
bool read_all(int fd, void* buf, size_t n, uint64_t off) {
  uint8_t* p = static_cast<uint8_t*>(buf);
  while (n > 0) {
    ssize_t r = pread(fd, p, n, (off_t)off);
    if (r <= 0) return false;
    p += r; n -= (size_t)r; off += (uint64_t)r;
  }
  return true;
}

// parallel pwrite / pread of one large payload
template <bool kWrite>
bool parallel_io(int fd, void* buf, uint64_t n, uint64_t off) {
  const uint64_t kChunk = 32ull << 20;
  if (n <= kChunk) return kWrite ? write_all(fd, buf, n, off) : read_all(fd, buf, n, off);
  unsigned nt = std::thread::hardware_concurrency();
  if (nt == 0) nt = 4;
  if (nt > 8) nt = 8;
  uint64_t per = (n + nt - 1) / nt;
  per = (per + 4095) & ~4095ull;
  std::vector<std::thread> th;
  std::vector<char> ok(nt, 1);
  for (unsigned t = 0; t < nt; ++t) {
    const uint64_t a = t * per;
    if (a >= n) break;
    const uint64_t len = (a + per <= n) ? per : n - a;
    th.emplace_back([=, &ok] {
      uint8_t* p = static_cast<uint8_t*>(buf) + a;
      ok[t] = kWrite ? write_all(fd, p, len, off + a) : read_all(fd, p, len, off + a);
    });
  }
  for (auto& x : th) x.join();
  for (char c : ok)
    if (!c) return false;
  return true;
}

}  // namespace

extern "C" {

void* lbh_writer_open(const char* path) {
  int fd = open(path, O_CREAT | O_TRUNC | O_WRONLY, 0644);
  if (fd < 0) return nullptr;
  Writer* w = new Writer;
  w->fd = fd;
  uint8_t hdr[16] = {'L', 'B', 'T', '1', 1, 0, 0, 0, 0, 0, 0, 0, 0, 0, 0, 0};
  if (!write_all(fd, hdr, 16, 0)) { close(fd); delete w; return nullptr; }
  w->pos = 16;
  return w;
}

int lbh_writer_add(void* handle, const char* name, uint32_t dtype, uint32_t ndim,
                   const uint64_t* dims, const void* data, uint64_t nbytes) {
  Writer* w = static_cast<Writer*>(handle);
  if (!w || ndim > 8) return -1;
  const uint32_t name_len = (uint32_t)strlen(name);
  std::vector<uint8_t> head;
  auto put = [&](const void* p, size_t n) {
    const uint8_t* b = static_cast<const uint8_t*>(p);
    head.insert(head.end(), b, b + n);
  };
  put(&name_len, 4); put(name, name_len); put(&dtype, 4); put(&ndim, 4);
  put(dims, 8 * ndim); put(&nbytes, 8);
  const uint32_t crc = crc32(static_cast<const uint8_t*>(data), nbytes);
  put(&crc, 4);
  uint64_t data_off = (w->pos + head.size() + 63) & ~63ull;
  std::vector<uint8_t> pad(data_off - (w->pos + head.size()), 0);
  if (!write_all(w->fd, head.data(), head.size(), w->pos)) return -2;
  if (!pad.empty() && !write_all(w->fd, pad.data(), pad.size(), w->pos + head.size())) return -2;
  if (nbytes && !parallel_io<true>(w->fd, const_cast<void*>(data), nbytes, data_off)) return -2;
  w->pos = data_off + nbytes;
  w->count += 1;
  return 0;
}

int lbh_writer_close(void* handle) {
  Writer* w = static_cast<Writer*>(handle);
  if (!w) return -1;
  bool ok = write_all(w->fd, &w->count, 8, 8);
  ok = ok && fsync(w->fd) == 0;
  close(w->fd);
  delete w;
  return ok ? 0 : -2;
}

void* lbh_reader_open(const char* path) {
  int fd = open(path, O_RDONLY);
  if (fd < 0) return nullptr;
  uint8_t hdr[16];
  if (!read_all(fd, hdr, 16, 0) || memcmp(hdr, "LBT1", 4) != 0) { close(fd); return nullptr; }
  uint64_t count;
  memcpy(&count, hdr + 8, 8);
  Reader* r = new Reader;
  r->fd = fd;
  uint64_t pos = 16;
  for (uint64_t i = 0; i < count; ++i) {
    Entry e;
    uint32_t name_len;
    if (!read_all(fd, &name_len, 4, pos) || name_len > (1u << 20)) { close(fd); delete r; return nullptr; }
    pos += 4;
    e.name.resize(name_len);
    if (name_len && !read_all(fd, &e.name[0], name_len, pos)) { close(fd); delete r; return nullptr; }
    pos += name_len;
    uint32_t two[2];
    if (!read_all(fd, two, 8, pos)) { close(fd); delete r; return nullptr; }
    pos += 8;
    e.dtype = two[0]; e.ndim = two[1];
    if (e.ndim > 8) { close(fd); delete r; return nullptr; }
    if (e.ndim && !read_all(fd, e.dims, 8 * e.ndim, pos)) { close(fd); delete r; return nullptr; }
    pos += 8 * e.ndim;
    if (!read_all(fd, &e.nbytes, 8, pos)) { close(fd); delete r; return nullptr; }
    pos += 8;
    if (!read_all(fd, &e.crc, 4, pos)) { close(fd); delete r; return nullptr; }
    pos += 4;
    e.offset = (pos + 63) & ~63ull;
    pos = e.offset + e.nbytes;
    r->entries.push_back(e);
  }
  return r;
}

long long lbh_reader_count(void* handle) {
  Reader* r = static_cast<Reader*>(handle);
  return r ? (long long)r->entries.size() : -1;
}

// name_buf must hold name_cap bytes; dims must hold 8 entries.
int lbh_reader_entry(void* handle, long long i, char* name_buf, int name_cap, uint32_t* dtype,
                     uint32_t* ndim, uint64_t* dims, uint64_t* nbytes) {
  Reader* r = static_cast<Reader*>(handle);
  if (!r || i < 0 || (size_t)i >= r->entries.size()) return -1;
  const Entry& e = r->entries[(size_t)i];
  if ((int)e.name.size() + 1 > name_cap) return -3;
  memcpy(name_buf, e.name.c_str(), e.name.size() + 1);
  *dtype = e.dtype; *ndim = e.ndim; *nbytes = e.nbytes;
  for (uint32_t k = 0; k < e.ndim; ++k) dims[k] = e.dims[k];
  return 0;
}

// Reads entry i into dst (nbytes of the entry) and verifies the checksum.
int lbh_reader_read(void* handle, long long i, void* dst) {
  Reader* r = static_cast<Reader*>(handle);
  if (!r || i < 0 || (size_t)i >= r->entries.size()) return -1;
  const Entry& e = r->entries[(size_t)i];
  if (e.nbytes && !parallel_io<false>(r->fd, dst, e.nbytes, e.offset)) return -2;
  if (crc32(static_cast<const uint8_t*>(dst), e.nbytes) != e.crc) return -4;
  return 0;
}

int lbh_reader_close(void* handle) {
  Reader* r = static_cast<Reader*>(handle);
  if (!r) return -1;
  close(r->fd);
  delete r;
  return 0;
}

// Collation: dst[i * row_bytes ...] = *srcs[i] for n rows, split over nthreads threads.
int lbh_gather_rows(void* dst, const void* const* srcs, long long n, long long row_bytes,
                    int nthreads) {
  if (n <= 0) return 0;
  if (nthreads < 1) nthreads = 1;
  if (nthreads > n) nthreads = (int)n;
  auto work = [=](long long a, long long b) {
    for (long long i = a; i < b; ++i)
      memcpy(static_cast<uint8_t*>(dst) + i * row_bytes, srcs[i], (size_t)row_bytes);
  };
  if (nthreads == 1) { work(0, n); return 0; }
  std::vector<std::thread> th;
  const long long per = (n + nthreads - 1) / nthreads;
  for (int t = 0; t < nthreads; ++t) {
    const long long a = t * per, b = (a + per < n) ? a + per : n;
    if (a >= n) break;
    th.emplace_back(work, a, b);
  }
  for (auto& x : th) x.join();
  return 0;
}

// Kahn topological order of a DAG given as edge list (u -> v); nodes listed in `first`
// (flag per node) are emitted before other ready nodes.  Returns the number of nodes
// ordered (< n means a cycle).
int lbh_topo_sort(int n, int m, const int* eu, const int* ev, const unsigned char* first,
                  int* order) {
  std::vector<int> indeg(n, 0);
  std::vector<std::vector<int>> adj(n);
  for (int i = 0; i < m; ++i) { adj[eu[i]].push_back(ev[i]); indeg[ev[i]]++; }
  std::vector<int> ready;
  for (int pass = 0; pass < 2; ++pass)
    for (int i = 0; i < n; ++i)
      if (indeg[i] == 0 && ((first && first[i]) ? pass == 0 : pass == 1)) ready.push_back(i);
  int k = 0;
  size_t head = 0;
  while (head < ready.size()) {
    const int u = ready[head++];
    order[k++] = u;
    for (int v : adj[u])
      if (--indeg[v] == 0) ready.push_back(v);
  }
  return k;
}

}  // extern "C"
