// Memory-mapped token file reader: fixed-width token ids (uint16 or int32) in one flat file, windows of
// seq_len + 1 tokens gathered into an int64 batch.  The native counterpart of the reference's MmapDataset
// (crates/data/src/lib.rs, memmap2) specialised for language-model pre-training data.
#include <fcntl.h>
#include <string.h>
#include <sys/mman.h>
#include <sys/stat.h>
#include <unistd.h>

#include "rb_runtime.h"

struct RbTokenFile {
  int fd;
  const uint8_t* base;
  size_t bytes;
  int width;
};

static inline uint64_t splitmix64(uint64_t& x) {
  uint64_t z = (x += 0x9E3779B97F4A7C15ull);
  z = (z ^ (z >> 30)) * 0xBF58476D1CE4E5B9ull;
  z = (z ^ (z >> 27)) * 0x94D049BB133111EBull;
  return z ^ (z >> 31);
}

extern "C" {

RbTokenFile* rb_tokens_open(const char* path, int bytes_per_token) {
  if (bytes_per_token != 2 && bytes_per_token != 4) return nullptr;
  const int fd = open(path, O_RDONLY);
  if (fd < 0) return nullptr;
  struct stat st;
  if (fstat(fd, &st) != 0 || st.st_size < bytes_per_token) { close(fd); return nullptr; }
  void* p = mmap(nullptr, (size_t)st.st_size, PROT_READ, MAP_PRIVATE, fd, 0);
  if (p == MAP_FAILED) { close(fd); return nullptr; }
  madvise(p, (size_t)st.st_size, MADV_RANDOM);
  auto* f = new RbTokenFile{fd, (const uint8_t*)p, (size_t)st.st_size, bytes_per_token};
  return f;
}
void rb_tokens_close(RbTokenFile* f) {
  if (!f) return;
  munmap((void*)f->base, f->bytes);
  close(f->fd);
  delete f;
}
int64_t rb_tokens_len(const RbTokenFile* f) { return (int64_t)(f->bytes / (size_t)f->width); }

int rb_tokens_gather(const RbTokenFile* f, const int64_t* offsets, int batch, int n, int64_t* out) {
  const int64_t len = rb_tokens_len(f);
  for (int b = 0; b < batch; ++b) {
    const int64_t o = offsets[b];
    if (o < 0 || o + n > len) return -1;
    if (f->width == 2) {
      const uint16_t* p = (const uint16_t*)f->base + o;
      for (int i = 0; i < n; ++i) out[(int64_t)b * n + i] = p[i];
    } else {
      const int32_t* p = (const int32_t*)f->base + o;
      for (int i = 0; i < n; ++i) out[(int64_t)b * n + i] = p[i];
    }
  }
  return 0;
}

void rb_tokens_sample_offsets(const RbTokenFile* f, uint64_t seed, uint64_t step, int batch, int n, int64_t* out) {
  const int64_t span = rb_tokens_len(f) - n + 1;
  uint64_t st = seed * 0x9E3779B97F4A7C15ull + step * 0xD1B54A32D192ED03ull + 1;
  for (int b = 0; b < batch; ++b) out[b] = span > 0 ? (int64_t)(splitmix64(st) % (uint64_t)span) : 0;
}

}  // extern "C"
