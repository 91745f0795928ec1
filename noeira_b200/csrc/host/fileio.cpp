// Atomic chunked file writes (temp file + fsync + rename), ranged reads and SHA-256.
// Counterpart of the reference's chunked fileio / checkpoint writer (noeira/io/fileio.mojo; nn/core/checkpoint.mojo:326
// streams <= 1 GiB chunks and renames into place) and noeira/io/sha256.mojo.
#include <cerrno>
#include <cstdint>
#include <cstdio>
#include <cstring>
#include <fcntl.h>
#include <string>
#include <unistd.h>

#include "host_api.h"

namespace {
constexpr size_t CHUNK = (size_t)1 << 30;

inline uint32_t rotr(uint32_t x, int n) { return (x >> n) | (x << (32 - n)); }
const uint32_t K[64] = {
    0x428a2f98, 0x71374491, 0xb5c0fbcf, 0xe9b5dba5, 0x3956c25b, 0x59f111f1, 0x923f82a4, 0xab1c5ed5, 0xd807aa98, 0x12835b01,
    0x243185be, 0x550c7dc3, 0x72be5d74, 0x80deb1fe, 0x9bdc06a7, 0xc19bf174, 0xe49b69c1, 0xefbe4786, 0x0fc19dc6, 0x240ca1cc,
    0x2de92c6f, 0x4a7484aa, 0x5cb0a9dc, 0x76f988da, 0x983e5152, 0xa831c66d, 0xb00327c8, 0xbf597fc7, 0xc6e00bf3, 0xd5a79147,
    0x06ca6351, 0x14292967, 0x27b70a85, 0x2e1b2138, 0x4d2c6dfc, 0x53380d13, 0x650a7354, 0x766a0abb, 0x81c2c92e, 0x92722c85,
    0xa2bfe8a1, 0xa81a664b, 0xc24b8b70, 0xc76c51a3, 0xd192e819, 0xd6990624, 0xf40e3585, 0x106aa070, 0x19a4c116, 0x1e376c08,
    0x2748774c, 0x34b0bcb5, 0x391c0cb3, 0x4ed8aa4a, 0x5b9cca4f, 0x682e6ff3, 0x748f82ee, 0x78a5636f, 0x84c87814, 0x8cc70208,
    0x90befffa, 0xa4506ceb, 0xbef9a3f7, 0xc67178f2};

void sha_block(uint32_t h[8], const uint8_t* b) {
  uint32_t w[64];
  for (int i = 0; i < 16; ++i) w[i] = (uint32_t)b[4 * i] << 24 | (uint32_t)b[4 * i + 1] << 16 | (uint32_t)b[4 * i + 2] << 8 | b[4 * i + 3];
  for (int i = 16; i < 64; ++i) {
    const uint32_t s0 = rotr(w[i - 15], 7) ^ rotr(w[i - 15], 18) ^ (w[i - 15] >> 3);
    const uint32_t s1 = rotr(w[i - 2], 17) ^ rotr(w[i - 2], 19) ^ (w[i - 2] >> 10);
    w[i] = w[i - 16] + s0 + w[i - 7] + s1;
  }
  uint32_t a = h[0], bb = h[1], c = h[2], d = h[3], e = h[4], f = h[5], g = h[6], hh = h[7];
  for (int i = 0; i < 64; ++i) {
    const uint32_t S1 = rotr(e, 6) ^ rotr(e, 11) ^ rotr(e, 25), ch = (e & f) ^ (~e & g), t1 = hh + S1 + ch + K[i] + w[i];
    const uint32_t S0 = rotr(a, 2) ^ rotr(a, 13) ^ rotr(a, 22), mj = (a & bb) ^ (a & c) ^ (bb & c), t2 = S0 + mj;
    hh = g; g = f; f = e; e = d + t1; d = c; c = bb; bb = a; a = t1 + t2;
  }
  h[0] += a; h[1] += bb; h[2] += c; h[3] += d; h[4] += e; h[5] += f; h[6] += g; h[7] += hh;
}
}  // namespace

extern "C" {

int nbh_write_file_atomic(const char* path, const void* const* chunks, const size_t* sizes, int n_chunks) {
  const std::string tmp = std::string(path) + ".tmp." + std::to_string((long)getpid());
  const int fd = open(tmp.c_str(), O_WRONLY | O_CREAT | O_TRUNC, 0644);
  if (fd < 0) return -errno;
  for (int i = 0; i < n_chunks; ++i) {
    const uint8_t* p = (const uint8_t*)chunks[i];
    size_t left = sizes[i];
    while (left) {
      const size_t n = left < CHUNK ? left : CHUNK;
      const ssize_t w = write(fd, p, n);
      if (w < 0) { if (errno == EINTR) continue; const int e = errno; close(fd); unlink(tmp.c_str()); return -e; }
      p += w; left -= (size_t)w;
    }
  }
  if (fsync(fd) != 0) { const int e = errno; close(fd); unlink(tmp.c_str()); return -e; }
  close(fd);
  if (rename(tmp.c_str(), path) != 0) { const int e = errno; unlink(tmp.c_str()); return -e; }
  return 0;
}

int64_t nbh_read_file_range(const char* path, uint64_t offset, void* out, size_t n) {
  const int fd = open(path, O_RDONLY);
  if (fd < 0) return -errno;
  size_t done = 0;
  while (done < n) {
    const ssize_t r = pread(fd, (uint8_t*)out + done, n - done < CHUNK ? n - done : CHUNK, (off_t)(offset + done));
    if (r < 0) { if (errno == EINTR) continue; const int e = errno; close(fd); return -e; }
    if (r == 0) break;
    done += (size_t)r;
  }
  close(fd);
  return (int64_t)done;
}

int nbh_sha256(const void* data, size_t n, uint8_t out32[32]) {
  uint32_t h[8] = {0x6a09e667, 0xbb67ae85, 0x3c6ef372, 0xa54ff53a, 0x510e527f, 0x9b05688c, 0x1f83d9ab, 0x5be0cd19};
  const uint8_t* p = (const uint8_t*)data;
  size_t i = 0;
  for (; i + 64 <= n; i += 64) sha_block(h, p + i);
  uint8_t tail[128];
  const size_t rem = n - i;
  memcpy(tail, p + i, rem);
  tail[rem] = 0x80;
  const size_t padded = rem + 1 + 8 <= 64 ? 64 : 128;
  memset(tail + rem + 1, 0, padded - rem - 1);
  const uint64_t bits = (uint64_t)n * 8;
  for (int k = 0; k < 8; ++k) tail[padded - 1 - k] = (uint8_t)(bits >> (8 * k));
  sha_block(h, tail);
  if (padded == 128) sha_block(h, tail + 64);
  for (int k = 0; k < 8; ++k) { out32[4 * k] = h[k] >> 24; out32[4 * k + 1] = h[k] >> 16; out32[4 * k + 2] = h[k] >> 8; out32[4 * k + 3] = h[k]; }
  return 0;
}

}  // extern "C"
