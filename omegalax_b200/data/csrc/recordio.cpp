// Indexed record file ("OLRF"): random-access container for the SFT datasets.
//
//   [8]  magic "OLRF0001"
//   n x  { u32 length, u32 crc32, bytes[length] }
//   n x  u64 absolute offset of record i
//   [8]  u64 n   [8] u64 offset of the offset table   [8] magic "OLRFIDX1"
//
// The reader memory-maps the file; reads are zero-copy pointer lookups plus an optional
// CRC check, and `olrf_read_many` gathers a batch of records with a small thread pool so the
// Python data loader spends no time in the interpreter per record.
#include <fcntl.h>
#include <stdint.h>
#include <stdio.h>
#include <string.h>
#include <sys/mman.h>
#include <sys/stat.h>
#include <unistd.h>

#include <atomic>
#include <thread>
#include <vector>

namespace {

const char kMagic[8] = {'O', 'L', 'R', 'F', '0', '0', '0', '1'};
const char kIdxMagic[8] = {'O', 'L', 'R', 'F', 'I', 'D', 'X', '1'};

uint32_t crc_table[256];
std::atomic<bool> crc_ready{false};

void init_crc() {
  if (crc_ready.load()) return;
  for (uint32_t i = 0; i < 256; ++i) {
    uint32_t c = i;
    for (int k = 0; k < 8; ++k) c = (c & 1) ? (0xEDB88320u ^ (c >> 1)) : (c >> 1);
    crc_table[i] = c;
  }
  crc_ready.store(true);
}

uint32_t crc32(const uint8_t* p, size_t n) {
  init_crc();
  uint32_t c = 0xFFFFFFFFu;
  for (size_t i = 0; i < n; ++i) c = crc_table[(c ^ p[i]) & 0xFF] ^ (c >> 8);
  return c ^ 0xFFFFFFFFu;
}

struct Reader {
  int fd = -1;
  const uint8_t* base = nullptr;
  size_t size = 0;
  uint64_t n = 0;
  const uint64_t* offsets = nullptr;
};

struct Writer {
  FILE* f = nullptr;
  std::vector<uint64_t> offsets;
  uint64_t pos = 0;
};

}  // namespace

extern "C" {

void* olrf_open(const char* path) {
  Reader* r = new Reader();
  r->fd = open(path, O_RDONLY);
  if (r->fd < 0) { delete r; return nullptr; }
  struct stat st;
  if (fstat(r->fd, &st) != 0 || st.st_size < 32) { close(r->fd); delete r; return nullptr; }
  r->size = (size_t)st.st_size;
  void* m = mmap(nullptr, r->size, PROT_READ, MAP_PRIVATE, r->fd, 0);
  if (m == MAP_FAILED) { close(r->fd); delete r; return nullptr; }
  r->base = (const uint8_t*)m;
  if (memcmp(r->base, kMagic, 8) != 0 || memcmp(r->base + r->size - 8, kIdxMagic, 8) != 0) {
    munmap(m, r->size); close(r->fd); delete r; return nullptr;
  }
  uint64_t n, table;
  memcpy(&n, r->base + r->size - 24, 8);
  memcpy(&table, r->base + r->size - 16, 8);
  if (table + n * 8 + 24 != r->size) { munmap(m, r->size); close(r->fd); delete r; return nullptr; }
  r->n = n;
  r->offsets = (const uint64_t*)(r->base + table);
  return r;
}

void olrf_close(void* h) {
  Reader* r = (Reader*)h;
  if (!r) return;
  if (r->base) munmap((void*)r->base, r->size);
  if (r->fd >= 0) close(r->fd);
  delete r;
}

long long olrf_num_records(void* h) { return h ? (long long)((Reader*)h)->n : -1; }

long long olrf_record_len(void* h, long long i) {
  Reader* r = (Reader*)h;
  if (!r || i < 0 || (uint64_t)i >= r->n) return -1;
  uint32_t len;
  memcpy(&len, r->base + r->offsets[i], 4);
  return len;
}

// Copies record i into dst (capacity cap).  Returns its length, -1 on a bad index,
// -2 if dst is too small, -3 on a checksum mismatch (only when verify != 0).
long long olrf_read(void* h, long long i, uint8_t* dst, long long cap, int verify) {
  Reader* r = (Reader*)h;
  if (!r || i < 0 || (uint64_t)i >= r->n) return -1;
  const uint8_t* p = r->base + r->offsets[i];
  uint32_t len, crc;
  memcpy(&len, p, 4);
  memcpy(&crc, p + 4, 4);
  if ((long long)len > cap) return -2;
  if (verify && crc32(p + 8, len) != crc) return -3;
  memcpy(dst, p + 8, len);
  return len;
}

// Gathers `count` records into one contiguous buffer; out_offsets[count+1] receives the
// boundaries.  Returns total bytes or a negative error as in olrf_read.
long long olrf_read_many(void* h, const long long* idx, int count, uint8_t* dst, long long cap,
                         long long* out_offsets, int verify, int threads) {
  Reader* r = (Reader*)h;
  if (!r) return -1;
  long long total = 0;
  out_offsets[0] = 0;
  for (int k = 0; k < count; ++k) {
    long long len = olrf_record_len(h, idx[k]);
    if (len < 0) return -1;
    total += len;
    out_offsets[k + 1] = total;
  }
  if (total > cap) return -2;
  std::atomic<int> next{0};
  std::atomic<long long> err{0};
  auto work = [&]() {
    for (;;) {
      int k = next.fetch_add(1);
      if (k >= count) break;
      long long rc = olrf_read(h, idx[k], dst + out_offsets[k], out_offsets[k + 1] - out_offsets[k], verify);
      if (rc < 0) err.store(rc);
    }
  };
  int nt = threads < 1 ? 1 : (threads > 16 ? 16 : threads);
  if (nt == 1 || count < 4) {
    work();
  } else {
    std::vector<std::thread> pool;
    for (int t = 0; t < nt; ++t) pool.emplace_back(work);
    for (auto& t : pool) t.join();
  }
  return err.load() < 0 ? err.load() : total;
}

void* olrf_writer_open(const char* path) {
  Writer* w = new Writer();
  w->f = fopen(path, "wb");
  if (!w->f) { delete w; return nullptr; }
  fwrite(kMagic, 1, 8, w->f);
  w->pos = 8;
  return w;
}

int olrf_writer_append(void* h, const uint8_t* data, long long len) {
  Writer* w = (Writer*)h;
  if (!w || len < 0 || len > 0xFFFFFFFFll) return -1;
  uint32_t l = (uint32_t)len, c = crc32(data, (size_t)len);
  w->offsets.push_back(w->pos);
  if (fwrite(&l, 4, 1, w->f) != 1 || fwrite(&c, 4, 1, w->f) != 1) return -2;
  if (len && fwrite(data, 1, (size_t)len, w->f) != (size_t)len) return -2;
  w->pos += 8 + (uint64_t)len;
  return 0;
}

int olrf_writer_close(void* h) {
  Writer* w = (Writer*)h;
  if (!w) return -1;
  uint64_t table = w->pos, n = w->offsets.size();
  if (n) fwrite(w->offsets.data(), 8, n, w->f);
  fwrite(&n, 8, 1, w->f);
  fwrite(&table, 8, 1, w->f);
  fwrite(kIdxMagic, 1, 8, w->f);
  int rc = fclose(w->f);
  delete w;
  return rc;
}

}  // extern "C"
