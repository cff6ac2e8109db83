// Host-side helpers with a plain C ABI (loaded through ctypes, no CUDA, no torch):
//   * xv_hash_chain      - chained XXH64 page hashes for the prefix cache
//   * xv_fill_decode     - per-step decode metadata (positions, slots, lengths, table rows)
//   * xv_fill_slots      - KV slot ids for a token range of one sequence
//   * xv_st_*            - safetensors header parsing and strided row/column reads via mmap
// The reference has no native code; it calls the xxhash and safetensors wheels for the
// first and last of these (reference: src/data/prefix/hash_util.py:16-30,
// src/compute/models/loader.py:55-76) and builds the decode metadata in a Python loop
// (reference: src/compute/batch.py:111-136).

#include <cstdint>
#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <string>
#include <vector>

#include <fcntl.h>
#include <sys/mman.h>
#include <sys/stat.h>
#include <unistd.h>

namespace {

constexpr uint64_t P1 = 11400714785074694791ULL;
constexpr uint64_t P2 = 14029467366897019727ULL;
constexpr uint64_t P3 = 1609587929392839161ULL;
constexpr uint64_t P4 = 9650029242287828579ULL;
constexpr uint64_t P5 = 2870177450012600261ULL;

inline uint64_t rotl(uint64_t x, int r) { return (x << r) | (x >> (64 - r)); }
inline uint64_t rd64(const uint8_t* p) { uint64_t v; std::memcpy(&v, p, 8); return v; }
inline uint32_t rd32(const uint8_t* p) { uint32_t v; std::memcpy(&v, p, 4); return v; }
inline uint64_t lane_round(uint64_t acc, uint64_t in) { return rotl(acc + in * P2, 31) * P1; }
inline uint64_t lane_merge(uint64_t h, uint64_t v) { return (h ^ lane_round(0, v)) * P1 + P4; }

// XXH64 with seed 0 over a contiguous buffer (public xxHash specification).
uint64_t xxh64(const uint8_t* p, size_t len) {
  const uint8_t* const end = p + len;
  uint64_t h;
  if (len >= 32) {
    uint64_t v1 = P1 + P2, v2 = P2, v3 = 0, v4 = 0 - P1;
    const uint8_t* const limit = end - 32;
    do {
      v1 = lane_round(v1, rd64(p));
      v2 = lane_round(v2, rd64(p + 8));
      v3 = lane_round(v3, rd64(p + 16));
      v4 = lane_round(v4, rd64(p + 24));
      p += 32;
    } while (p <= limit);
    h = rotl(v1, 1) + rotl(v2, 7) + rotl(v3, 12) + rotl(v4, 18);
    h = lane_merge(h, v1); h = lane_merge(h, v2); h = lane_merge(h, v3); h = lane_merge(h, v4);
  } else {
    h = P5;
  }
  h += static_cast<uint64_t>(len);
  while (p + 8 <= end) { h = rotl(h ^ lane_round(0, rd64(p)), 27) * P1 + P4; p += 8; }
  if (p + 4 <= end) { h = rotl(h ^ (static_cast<uint64_t>(rd32(p)) * P1), 23) * P2 + P3; p += 4; }
  while (p < end) { h = rotl(h ^ (static_cast<uint64_t>(*p) * P5), 11) * P1; ++p; }
  h ^= h >> 33; h *= P2; h ^= h >> 29; h *= P3; h ^= h >> 32;
  return h;
}

struct StFile {
  int fd = -1;
  const uint8_t* base = nullptr;
  size_t size = 0;
  uint64_t header_len = 0;
};

}  // namespace

extern "C" {

// out[i] = XXH64(le64(out[i-1]) | tokens of page i); the parent is omitted for the first
// page when has_parent == 0.
void xv_hash_chain(const int32_t* tokens, int num_blocks, int block_size, uint64_t parent,
                   int has_parent, uint64_t* out) {
  std::vector<uint8_t> buf(8 + static_cast<size_t>(block_size) * 4);
  const size_t body = static_cast<size_t>(block_size) * 4;
  for (int i = 0; i < num_blocks; ++i) {
    const int32_t* src = tokens + static_cast<size_t>(i) * block_size;
    uint64_t h;
    if (has_parent) {
      std::memcpy(buf.data(), &parent, 8);
      std::memcpy(buf.data() + 8, src, body);
      h = xxh64(buf.data(), 8 + body);
    } else {
      h = xxh64(reinterpret_cast<const uint8_t*>(src), body);
    }
    out[i] = h;
    parent = h;
    has_parent = 1;
  }
}

uint64_t xv_xxh64(const uint8_t* data, uint64_t len) { return xxh64(data, len); }

// KV slots of positions [start, end) given a block table.
void xv_fill_slots(const int32_t* block_table, int start, int end, int block_size, int32_t* out) {
  for (int p = start; p < end; ++p)
    out[p - start] = block_table[p / block_size] * block_size + p % block_size;
}

// Decode metadata for n sequences. rows[i] selects a row of the persistent host block
// table `tables` (row stride `max_blocks`); cached[i] is the KV length before this step.
// Writes positions, slot of the new token, kv length after the step, and copies each
// sequence's live block-table prefix into `bt_out` (row stride `bt_stride`, zero padded).
void xv_fill_decode(int n, const int32_t* rows, const int32_t* cached, const int32_t* tables,
                    int max_blocks, int block_size, int32_t* positions, int32_t* slots,
                    int32_t* kv_lens, int32_t* bt_out, int bt_stride) {
  for (int i = 0; i < n; ++i) {
    const int32_t* t = tables + static_cast<size_t>(rows[i]) * max_blocks;
    const int pos = cached[i];
    positions[i] = pos;
    slots[i] = t[pos / block_size] * block_size + pos % block_size;
    kv_lens[i] = pos + 1;
    const int nb = pos / block_size + 1;
    int32_t* o = bt_out + static_cast<size_t>(i) * bt_stride;
    std::memcpy(o, t, static_cast<size_t>(nb) * 4);
    if (bt_stride > nb) std::memset(o + nb, 0, static_cast<size_t>(bt_stride - nb) * 4);
  }
}

// ---- safetensors: [u64 header_len][JSON header][raw tensor bytes] -------------------------
// The JSON is parsed in Python (it is tiny); this side only maps the file and copies
// strided sub-blocks so a rank reads just the rows/columns it owns.

void* xv_st_open(const char* path) {
  int fd = ::open(path, O_RDONLY);
  if (fd < 0) return nullptr;
  struct stat st;
  if (fstat(fd, &st) != 0 || st.st_size < 8) { ::close(fd); return nullptr; }
  void* m = mmap(nullptr, static_cast<size_t>(st.st_size), PROT_READ, MAP_PRIVATE, fd, 0);
  if (m == MAP_FAILED) { ::close(fd); return nullptr; }
  auto* f = new StFile;
  f->fd = fd;
  f->base = static_cast<const uint8_t*>(m);
  f->size = static_cast<size_t>(st.st_size);
  std::memcpy(&f->header_len, f->base, 8);
  if (f->header_len > f->size - 8) {
    munmap(m, f->size); ::close(fd); delete f; return nullptr;
  }
  return f;
}

uint64_t xv_st_header_len(void* h) { return static_cast<StFile*>(h)->header_len; }
uint64_t xv_st_file_size(void* h) { return static_cast<StFile*>(h)->size; }

// Copies the JSON header into `out` (capacity `cap`); returns bytes needed.
uint64_t xv_st_header(void* h, char* out, uint64_t cap) {
  auto* f = static_cast<StFile*>(h);
  if (cap >= f->header_len) std::memcpy(out, f->base + 8, f->header_len);
  return f->header_len;
}

// Reads rows [row0, row0+nrows) and byte columns [col0_bytes, col0_bytes+ncol_bytes) of a
// 2-D tensor stored at data offset `begin` with `row_bytes` per row. Returns 0 on success,
// -1 if the request leaves the file.
int xv_st_read_block(void* h, uint64_t begin, uint64_t row_bytes, uint64_t row0, uint64_t nrows,
                     uint64_t col0_bytes, uint64_t ncol_bytes, void* dst) {
  auto* f = static_cast<StFile*>(h);
  const uint64_t data0 = 8 + f->header_len + begin;
  if (ncol_bytes == 0 || nrows == 0) return 0;
  if (col0_bytes + ncol_bytes > row_bytes) return -1;
  const uint64_t last = data0 + (row0 + nrows - 1) * row_bytes + col0_bytes + ncol_bytes;
  if (last > f->size) return -1;
  auto* d = static_cast<uint8_t*>(dst);
  if (ncol_bytes == row_bytes) {
    std::memcpy(d, f->base + data0 + row0 * row_bytes, nrows * row_bytes);
    return 0;
  }
  for (uint64_t r = 0; r < nrows; ++r)
    std::memcpy(d + r * ncol_bytes, f->base + data0 + (row0 + r) * row_bytes + col0_bytes, ncol_bytes);
  return 0;
}

void xv_st_close(void* h) {
  auto* f = static_cast<StFile*>(h);
  if (!f) return;
  munmap(const_cast<uint8_t*>(f->base), f->size);
  ::close(f->fd);
  delete f;
}

}  // extern "C"
