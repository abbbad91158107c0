// Host-side runtime pieces that are hot enough to leave Python:
//
//   tf_host_sha256            one digest
//   tf_host_sha256_chunks     one digest per fixed-size chunk of a buffer, computed by a pool of
//                             threads and written in chunk order (state images, staged atlases)
//   tf_host_write_direct /    snapshot-tier file I/O that bypasses the page cache (O_DIRECT with a
//   tf_host_read_direct       4 KiB-aligned bounce buffer; falls back to buffered I/O where the
//                             filesystem refuses O_DIRECT), fsync before returning from a write
//   tf_host_frame_encode /    the control channel's frame: magic, kind, sequence, length, payload,
//   tf_host_frame_decode      CRC-32 of everything before it
// (reference: src/ordered_digest.rs, src/ordered_read_hash.rs in-order parallel SHA-256;
//  src/disk_tier.rs:20-22 chunking, :121 PendingWrite, :160 read; src/control_channel.rs:15-24 frames).
#include <fcntl.h>
#include <unistd.h>

#include <algorithm>
#include <atomic>
#include <cerrno>
#include <cstdint>
#include <cstdlib>
#include <cstring>
#include <thread>
#include <vector>

#define TF_API extern "C" __attribute__((visibility("default")))

namespace {

// ---------------------------------------------------------------------------- SHA-256 (FIPS 180-4)
const uint32_t K[64] = {
    0x428a2f98, 0x71374491, 0xb5c0fbcf, 0xe9b5dba5, 0x3956c25b, 0x59f111f1, 0x923f82a4, 0xab1c5ed5, 0xd807aa98,
    0x12835b01, 0x243185be, 0x550c7dc3, 0x72be5d74, 0x80deb1fe, 0x9bdc06a7, 0xc19bf174, 0xe49b69c1, 0xefbe4786,
    0x0fc19dc6, 0x240ca1cc, 0x2de92c6f, 0x4a7484aa, 0x5cb0a9dc, 0x76f988da, 0x983e5152, 0xa831c66d, 0xb00327c8,
    0xbf597fc7, 0xc6e00bf3, 0xd5a79147, 0x06ca6351, 0x14292967, 0x27b70a85, 0x2e1b2138, 0x4d2c6dfc, 0x53380d13,
    0x650a7354, 0x766a0abb, 0x81c2c92e, 0x92722c85, 0xa2bfe8a1, 0xa81a664b, 0xc24b8b70, 0xc76c51a3, 0xd192e819,
    0xd6990624, 0xf40e3585, 0x106aa070, 0x19a4c116, 0x1e376c08, 0x2748774c, 0x34b0bcb5, 0x391c0cb3, 0x4ed8aa4a,
    0x5b9cca4f, 0x682e6ff3, 0x748f82ee, 0x78a5636f, 0x84c87814, 0x8cc70208, 0x90befffa, 0xa4506ceb, 0xbef9a3f7,
    0xc67178f2};

inline uint32_t rotr(uint32_t x, int n) { return (x >> n) | (x << (32 - n)); }

struct Sha256 {
  uint32_t h[8] = {0x6a09e667, 0xbb67ae85, 0x3c6ef372, 0xa54ff53a, 0x510e527f, 0x9b05688c, 0x1f83d9ab, 0x5be0cd19};
  uint8_t buf[64];
  size_t fill = 0;
  uint64_t total = 0;

  void block(const uint8_t* p) {
    uint32_t w[64];
    for (int i = 0; i < 16; ++i)
      w[i] = (uint32_t)p[4 * i] << 24 | (uint32_t)p[4 * i + 1] << 16 | (uint32_t)p[4 * i + 2] << 8 | p[4 * i + 3];
    for (int i = 16; i < 64; ++i) {
      const uint32_t s0 = rotr(w[i - 15], 7) ^ rotr(w[i - 15], 18) ^ (w[i - 15] >> 3);
      const uint32_t s1 = rotr(w[i - 2], 17) ^ rotr(w[i - 2], 19) ^ (w[i - 2] >> 10);
      w[i] = w[i - 16] + s0 + w[i - 7] + s1;
    }
    uint32_t a = h[0], b = h[1], c = h[2], d = h[3], e = h[4], f = h[5], g = h[6], hh = h[7];
    for (int i = 0; i < 64; ++i) {
      const uint32_t t1 = hh + (rotr(e, 6) ^ rotr(e, 11) ^ rotr(e, 25)) + ((e & f) ^ (~e & g)) + K[i] + w[i];
      const uint32_t t2 = (rotr(a, 2) ^ rotr(a, 13) ^ rotr(a, 22)) + ((a & b) ^ (a & c) ^ (b & c));
      hh = g; g = f; f = e; e = d + t1; d = c; c = b; b = a; a = t1 + t2;
    }
    h[0] += a; h[1] += b; h[2] += c; h[3] += d; h[4] += e; h[5] += f; h[6] += g; h[7] += hh;
  }
  void update(const uint8_t* p, size_t n) {
    total += n;
    if (fill) {
      const size_t take = std::min(n, 64 - fill);
      memcpy(buf + fill, p, take);
      fill += take; p += take; n -= take;
      if (fill == 64) { block(buf); fill = 0; }
    }
    for (; n >= 64; p += 64, n -= 64) block(p);
    if (n) { memcpy(buf, p, n); fill = n; }
  }
  void finish(uint8_t out[32]) {
    const uint64_t bits = total * 8;
    const uint8_t one = 0x80, zero = 0;
    update(&one, 1);
    while (fill != 56) update(&zero, 1);
    uint8_t len[8];
    for (int i = 0; i < 8; ++i) len[i] = (uint8_t)(bits >> (56 - 8 * i));
    update(len, 8);
    for (int i = 0; i < 8; ++i)
      for (int j = 0; j < 4; ++j) out[4 * i + j] = (uint8_t)(h[i] >> (24 - 8 * j));
  }
};

uint32_t crc32(const uint8_t* p, size_t n) {
  static uint32_t table[256];
  static bool init = false;
  if (!init) {
    for (uint32_t i = 0; i < 256; ++i) {
      uint32_t c = i;
      for (int k = 0; k < 8; ++k) c = (c & 1) ? 0xEDB88320u ^ (c >> 1) : c >> 1;
      table[i] = c;
    }
    init = true;
  }
  uint32_t c = 0xFFFFFFFFu;
  for (size_t i = 0; i < n; ++i) c = table[(c ^ p[i]) & 0xFF] ^ (c >> 8);
  return c ^ 0xFFFFFFFFu;
}

constexpr size_t kAlign = 4096;
constexpr size_t kBounce = 8u << 20;
constexpr uint32_t kFrameMagic = 0x31465454u;   // "TTF1"

}  // namespace

TF_API int tf_host_sha256(const void* data, long n, void* out32) {
  Sha256 s;
  s.update((const uint8_t*)data, (size_t)n);
  s.finish((uint8_t*)out32);
  return 0;
}

// out: 32 bytes per chunk, ceil(n / chunk) chunks, in order
TF_API int tf_host_sha256_chunks(const void* data, long n, long chunk, void* out, int threads) {
  if (n < 0 || chunk <= 0) return -1;
  const long count = (n + chunk - 1) / chunk;
  std::atomic<long> next{0};
  auto work = [&]() {
    for (long i = next.fetch_add(1); i < count; i = next.fetch_add(1)) {
      Sha256 s;
      s.update((const uint8_t*)data + i * chunk, (size_t)std::min(chunk, n - i * chunk));
      s.finish((uint8_t*)out + 32 * i);
    }
  };
  threads = (int)std::max(1L, std::min<long>(threads, count));
  std::vector<std::thread> pool;
  for (int t = 1; t < threads; ++t) pool.emplace_back(work);
  work();
  for (auto& t : pool) t.join();
  return 0;
}

// returns bytes written, or -errno
TF_API long tf_host_write_direct(const char* path, const void* data, long n, int use_direct) {
  int fd = -1;
  if (use_direct) fd = open(path, O_WRONLY | O_CREAT | O_TRUNC | O_DIRECT, 0600);
  const bool direct = fd >= 0;
  if (fd < 0) fd = open(path, O_WRONLY | O_CREAT | O_TRUNC, 0600);
  if (fd < 0) return -errno;
  void* bounce = nullptr;
  if (posix_memalign(&bounce, kAlign, kBounce) != 0) { close(fd); return -ENOMEM; }
  long done = 0;
  int err = 0;
  while (done < n && !err) {
    const size_t take = (size_t)std::min<long>(kBounce, n - done);
    size_t padded = direct ? (take + kAlign - 1) / kAlign * kAlign : take;
    memcpy(bounce, (const uint8_t*)data + done, take);
    if (padded > take) memset((uint8_t*)bounce + take, 0, padded - take);
    size_t off = 0;
    while (off < padded) {
      const ssize_t w = write(fd, (uint8_t*)bounce + off, padded - off);
      if (w < 0) { if (errno == EINTR) continue; err = errno; break; }
      off += (size_t)w;
    }
    done += (long)take;
  }
  if (!err && direct && ftruncate(fd, n) != 0) err = errno;       // drop the alignment padding
  if (!err && fsync(fd) != 0) err = errno;
  free(bounce);
  close(fd);
  return err ? -err : done;
}

// returns bytes read (== n on success), or -errno; -EIO on a short file
TF_API long tf_host_read_direct(const char* path, void* out, long n, long offset, int use_direct) {
  int fd = -1;
  const bool aligned_off = offset % (long)kAlign == 0;
  if (use_direct && aligned_off) fd = open(path, O_RDONLY | O_DIRECT);
  const bool direct = fd >= 0;
  if (fd < 0) fd = open(path, O_RDONLY);
  if (fd < 0) return -errno;
  void* bounce = nullptr;
  if (posix_memalign(&bounce, kAlign, kBounce) != 0) { close(fd); return -ENOMEM; }
  long done = 0;
  int err = 0;
  while (done < n && !err) {
    const size_t want = (size_t)std::min<long>(kBounce, n - done);
    const size_t ask = direct ? (want + kAlign - 1) / kAlign * kAlign : want;
    const ssize_t r = pread(fd, bounce, ask, offset + done);
    if (r < 0) { if (errno == EINTR) continue; err = errno; break; }
    if (r == 0) { err = EIO; break; }
    const size_t got = std::min(want, (size_t)r);
    memcpy((uint8_t*)out + done, bounce, got);
    done += (long)got;
  }
  free(bounce);
  close(fd);
  return err ? -err : done;
}

// Batched positional reads of fixed-size rows (the row store of the hashed n-gram memory lives on
// NVMe; a lookup needs a few hundred scattered 264-byte rows).  A pool of threads issues one pread
// per row into the caller's buffer, in id order within each thread's share; rows whose id is
// negative or beyond `rows_in_file` are zero-filled.  Returns the number of rows read from the
// file, or -errno (reference: the batched reader of src/engram_io.rs:209-329).
TF_API long tf_host_read_rows(const char* path, long header_bytes, long row_bytes, long rows_in_file, const long* ids,
                              long n, void* out, int threads) {
  if (!path || !ids || !out || row_bytes <= 0 || n < 0) return -EINVAL;
  const int fd = open(path, O_RDONLY);
  if (fd < 0) return -errno;
  if (threads < 1) threads = 1;
  if (threads > 32) threads = 32;
  if (n < 64) threads = 1;
  std::vector<long> got((size_t)threads, 0);
  std::vector<int> errs((size_t)threads, 0);
  auto work = [&](int t) {
    const long lo = n * t / threads, hi = n * (t + 1) / threads;
    for (long i = lo; i < hi; ++i) {
      uint8_t* dst = (uint8_t*)out + i * row_bytes;
      const long id = ids[i];
      if (id < 0 || id >= rows_in_file) {
        memset(dst, 0, (size_t)row_bytes);
        continue;
      }
      long done = 0;
      while (done < row_bytes) {
        const ssize_t r = pread(fd, dst + done, (size_t)(row_bytes - done), header_bytes + id * row_bytes + done);
        if (r < 0) { if (errno == EINTR) continue; errs[(size_t)t] = errno; return; }
        if (r == 0) { errs[(size_t)t] = EIO; return; }
        done += (long)r;
      }
      got[(size_t)t] += 1;
    }
  };
  std::vector<std::thread> pool;
  for (int t = 1; t < threads; ++t) pool.emplace_back(work, t);
  work(0);
  for (auto& th : pool) th.join();
  close(fd);
  long total = 0;
  for (int t = 0; t < threads; ++t) {
    if (errs[(size_t)t]) return -errs[(size_t)t];
    total += got[(size_t)t];
  }
  return total;
}

// frame = magic u32 | kind u32 | seq u64 | len u32 | payload | crc32 u32   (little endian)
TF_API long tf_host_frame_bytes(long payload) { return 24 + payload; }
TF_API long tf_host_frame_encode(int kind, long seq, const void* payload, long n, void* out) {
  uint8_t* o = (uint8_t*)out;
  const uint32_t k = (uint32_t)kind, len = (uint32_t)n;
  const uint64_t s = (uint64_t)seq;
  memcpy(o, &kFrameMagic, 4); memcpy(o + 4, &k, 4); memcpy(o + 8, &s, 8); memcpy(o + 16, &len, 4);
  if (n) memcpy(o + 20, payload, (size_t)n);
  const uint32_t c = crc32(o, 20 + (size_t)n);
  memcpy(o + 20 + n, &c, 4);
  return 24 + n;
}
// returns payload length and fills kind / seq, or -1 bad magic, -2 truncated, -3 checksum
TF_API long tf_host_frame_decode(const void* frame, long n, int* kind, long* seq, void* payload_out, long cap) {
  const uint8_t* f = (const uint8_t*)frame;
  if (n < 24) return -2;
  uint32_t magic, k, len;
  uint64_t s;
  memcpy(&magic, f, 4); memcpy(&k, f + 4, 4); memcpy(&s, f + 8, 8); memcpy(&len, f + 16, 4);
  if (magic != kFrameMagic) return -1;
  if ((long)len + 24 > n || (long)len > cap) return -2;
  uint32_t c;
  memcpy(&c, f + 20 + len, 4);
  if (c != crc32(f, 20 + (size_t)len)) return -3;
  if (len) memcpy(payload_out, f + 20, len);
  *kind = (int)k;
  *seq = (long)s;
  return (long)len;
}
