// Multi-shard checkpoint I/O: one binary shard file per rank plus a JSON manifest written by the
// Python layer. Shard layout (little-endian), matching the reference's writer
// (src/MLFramework/Checkpointing/Formats/MultiShardCheckpointFormat.cs:111-183):
//     int32  magic 0x53484152 ("SHAR")
//     int32  rank
//     int32  checksum length, then that many UTF-8 bytes (hex SHA-256 of the payload)
//     int32  tensor count
//     int32  payload length   (-1 when the payload is 2 GiB or larger, followed by int64 length)
//     bytes  payload = the tensors' raw bytes back to back (offsets are in the manifest)
// Writes go to "<path>.tmp" and are renamed into place (the reference's atomic commit,
// Checkpointing/Coordinator/AtomicCommitProtocol.cs:25-100). SHA-256 is implemented here so the
// library has no external dependency.
#include <errno.h>
#include <stdint.h>
#include <stdio.h>
#include <string.h>
#include <unistd.h>

#include <string>
#include <vector>

#include "../common/host.h"

namespace mlf {

struct Sha256 {
  uint32_t h[8];
  uint64_t len = 0;
  uint8_t buf[64];
  size_t fill = 0;
  Sha256() {
    static const uint32_t init[8] = {0x6a09e667, 0xbb67ae85, 0x3c6ef372, 0xa54ff53a, 0x510e527f, 0x9b05688c, 0x1f83d9ab, 0x5be0cd19};
    memcpy(h, init, sizeof(h));
  }
  static uint32_t rotr(uint32_t x, int n) { return (x >> n) | (x << (32 - n)); }
  void block(const uint8_t* p) {
    static const uint32_t k[64] = {
        0x428a2f98, 0x71374491, 0xb5c0fbcf, 0xe9b5dba5, 0x3956c25b, 0x59f111f1, 0x923f82a4, 0xab1c5ed5, 0xd807aa98, 0x12835b01,
        0x243185be, 0x550c7dc3, 0x72be5d74, 0x80deb1fe, 0x9bdc06a7, 0xc19bf174, 0xe49b69c1, 0xefbe4786, 0x0fc19dc6, 0x240ca1cc,
        0x2de92c6f, 0x4a7484aa, 0x5cb0a9dc, 0x76f988da, 0x983e5152, 0xa831c66d, 0xb00327c8, 0xbf597fc7, 0xc6e00bf3, 0xd5a79147,
        0x06ca6351, 0x14292967, 0x27b70a85, 0x2e1b2138, 0x4d2c6dfc, 0x53380d13, 0x650a7354, 0x766a0abb, 0x81c2c92e, 0x92722c85,
        0xa2bfe8a1, 0xa81a664b, 0xc24b8b70, 0xc76c51a3, 0xd192e819, 0xd6990624, 0xf40e3585, 0x106aa070, 0x19a4c116, 0x1e376c08,
        0x2748774c, 0x34b0bcb5, 0x391c0cb3, 0x4ed8aa4a, 0x5b9cca4f, 0x682e6ff3, 0x748f82ee, 0x78a5636f, 0x84c87814, 0x8cc70208,
        0x90befffa, 0xa4506ceb, 0xbef9a3f7, 0xc67178f2};
    uint32_t w[64];
    for (int i = 0; i < 16; ++i) w[i] = (uint32_t)p[4 * i] << 24 | (uint32_t)p[4 * i + 1] << 16 | (uint32_t)p[4 * i + 2] << 8 | p[4 * i + 3];
    for (int i = 16; i < 64; ++i) {
      const uint32_t s0 = rotr(w[i - 15], 7) ^ rotr(w[i - 15], 18) ^ (w[i - 15] >> 3);
      const uint32_t s1 = rotr(w[i - 2], 17) ^ rotr(w[i - 2], 19) ^ (w[i - 2] >> 10);
      w[i] = w[i - 16] + s0 + w[i - 7] + s1;
    }
    uint32_t a = h[0], b = h[1], c = h[2], d = h[3], e = h[4], f = h[5], g = h[6], hh = h[7];
    for (int i = 0; i < 64; ++i) {
      const uint32_t S1 = rotr(e, 6) ^ rotr(e, 11) ^ rotr(e, 25);
      const uint32_t ch = (e & f) ^ (~e & g);
      const uint32_t t1 = hh + S1 + ch + k[i] + w[i];
      const uint32_t S0 = rotr(a, 2) ^ rotr(a, 13) ^ rotr(a, 22);
      const uint32_t mj = (a & b) ^ (a & c) ^ (b & c);
      const uint32_t t2 = S0 + mj;
      hh = g; g = f; f = e; e = d + t1; d = c; c = b; b = a; a = t1 + t2;
    }
    h[0] += a; h[1] += b; h[2] += c; h[3] += d; h[4] += e; h[5] += f; h[6] += g; h[7] += hh;
  }
  void update(const void* data, size_t n) {
    const uint8_t* p = static_cast<const uint8_t*>(data);
    len += n;
    if (fill) {
      const size_t take = n < 64 - fill ? n : 64 - fill;
      memcpy(buf + fill, p, take);
      fill += take; p += take; n -= take;
      if (fill == 64) { block(buf); fill = 0; }
    }
    while (n >= 64) { block(p); p += 64; n -= 64; }
    if (n) { memcpy(buf, p, n); fill = n; }
  }
  void hex(char out[65]) {
    const uint64_t bits = len * 8;
    uint8_t pad = 0x80;
    update(&pad, 1);
    const uint8_t zero = 0;
    while (fill != 56) update(&zero, 1);
    uint8_t lb[8];
    for (int i = 0; i < 8; ++i) lb[i] = (uint8_t)(bits >> (56 - 8 * i));
    update(lb, 8);
    static const char* d = "0123456789abcdef";
    for (int i = 0; i < 8; ++i)
      for (int j = 0; j < 4; ++j) {
        const uint8_t v = (uint8_t)(h[i] >> (24 - 8 * j));
        out[8 * i + 2 * j] = d[v >> 4];
        out[8 * i + 2 * j + 1] = d[v & 15];
      }
    out[64] = 0;
  }
};

constexpr int32_t kShardMagic = 0x53484152;

static bool write_all(FILE* f, const void* p, size_t n) { return n == 0 || fwrite(p, 1, n, f) == n; }

}  // namespace mlf

using namespace mlf;

MLF_API int mlf_sha256(const void* data, long long n, char* hex65) {
  Sha256 s;
  s.update(data, (size_t)n);
  s.hex(hex65);
  return 0;
}

MLF_API int mlf_sha256_file(const char* path, char* hex65) {
  FILE* f = fopen(path, "rb");
  MLF_REQUIRE(f != nullptr, "cannot open %s: %s", path, strerror(errno));
  Sha256 s;
  std::vector<uint8_t> buf(1 << 20);
  size_t n;
  while ((n = fread(buf.data(), 1, buf.size(), f)) > 0) s.update(buf.data(), n);
  fclose(f);
  s.hex(hex65);
  return 0;
}

// segs: n host pointers with their sizes, written back to back as the payload.
// checksum_out (65 bytes) receives the hex SHA-256 of the payload, which is also stored in the header.
MLF_API int mlf_ckpt_write_shard(const char* path, int rank, int tensor_count, const void* const* segs,
                                 const long long* sizes, int n, char* checksum_out, long long* file_size_out) {
  MLF_REQUIRE(path && n >= 0, "ckpt_write_shard: bad arguments");
  Sha256 sha;
  long long total = 0;
  for (int i = 0; i < n; ++i) {
    sha.update(segs[i], (size_t)sizes[i]);
    total += sizes[i];
  }
  char hex[65];
  sha.hex(hex);
  const std::string tmp = std::string(path) + ".tmp";
  FILE* f = fopen(tmp.c_str(), "wb");
  MLF_REQUIRE(f != nullptr, "cannot create %s: %s", tmp.c_str(), strerror(errno));
  const int32_t magic = kShardMagic, r = rank, cl = 64, tc = tensor_count;
  bool ok = write_all(f, &magic, 4) && write_all(f, &r, 4) && write_all(f, &cl, 4) && write_all(f, hex, 64) && write_all(f, &tc, 4);
  if (total < (1LL << 31)) {
    const int32_t dl = (int32_t)total;
    ok = ok && write_all(f, &dl, 4);
  } else {
    const int32_t dl = -1;
    const int64_t dl64 = total;
    ok = ok && write_all(f, &dl, 4) && write_all(f, &dl64, 8);
  }
  for (int i = 0; ok && i < n; ++i) ok = write_all(f, segs[i], (size_t)sizes[i]);
  ok = ok && fflush(f) == 0 && fsync(fileno(f)) == 0;
  const long long fsize = ftell(f);
  fclose(f);
  if (!ok) {
    remove(tmp.c_str());
    set_error("short write to %s: %s", tmp.c_str(), strerror(errno));
    return -3;
  }
  if (rename(tmp.c_str(), path) != 0) {
    set_error("cannot rename %s: %s", tmp.c_str(), strerror(errno));
    return -3;
  }
  if (checksum_out) memcpy(checksum_out, hex, 65);
  if (file_size_out) *file_size_out = fsize;
  return 0;
}

// Reads and validates the header. Return codes: 0 ok, -10 bad magic, -11 rank mismatch,
// -12 truncated. expected_rank < 0 skips the rank check.
MLF_API int mlf_ckpt_read_header(const char* path, int expected_rank, int* rank_out, char* checksum65, int* tensor_count,
                                 long long* data_len, long long* data_offset) {
  FILE* f = fopen(path, "rb");
  MLF_REQUIRE(f != nullptr, "cannot open %s: %s", path, strerror(errno));
  int32_t magic = 0, rank = 0, cl = 0, tc = 0, dl = 0;
  int rc = 0;
  char cs[256] = {0};
  if (fread(&magic, 4, 1, f) != 1) rc = -12;
  if (!rc && magic != kShardMagic) {
    set_error("invalid shard file %s: magic 0x%08X, expected 0x%08X", path, magic, kShardMagic);
    rc = -10;
  }
  if (!rc && fread(&rank, 4, 1, f) != 1) rc = -12;
  if (!rc && expected_rank >= 0 && rank != expected_rank) {
    set_error("shard rank mismatch in %s: expected %d, found %d", path, expected_rank, rank);
    rc = -11;
  }
  if (!rc && (fread(&cl, 4, 1, f) != 1 || cl < 0 || cl > 255 || fread(cs, 1, cl, f) != (size_t)cl)) rc = -12;
  if (!rc && fread(&tc, 4, 1, f) != 1) rc = -12;
  if (!rc && fread(&dl, 4, 1, f) != 1) rc = -12;
  long long total = dl;
  if (!rc && dl == -1) {
    int64_t d64 = 0;
    if (fread(&d64, 8, 1, f) != 1) rc = -12;
    total = d64;
  }
  if (rc == -12) set_error("truncated shard header in %s", path);
  if (!rc) {
    if (rank_out) *rank_out = rank;
    if (checksum65) { memcpy(checksum65, cs, cl < 64 ? cl : 64); checksum65[cl < 64 ? cl : 64] = 0; }
    if (tensor_count) *tensor_count = tc;
    if (data_len) *data_len = total;
    if (data_offset) *data_offset = ftell(f);
  }
  fclose(f);
  return rc;
}

// Reads `bytes` of payload starting at payload offset `offset` into dst (host memory).
MLF_API int mlf_ckpt_read_data(const char* path, long long data_offset, long long offset, long long bytes, void* dst) {
  FILE* f = fopen(path, "rb");
  MLF_REQUIRE(f != nullptr, "cannot open %s: %s", path, strerror(errno));
  int rc = 0;
  if (fseek(f, (long)(data_offset + offset), SEEK_SET) != 0 || fread(dst, 1, (size_t)bytes, f) != (size_t)bytes) {
    set_error("short read from %s", path);
    rc = -12;
  }
  fclose(f);
  return rc;
}

// SHA-256 of the payload only (what the header stores), for verification.
MLF_API int mlf_ckpt_payload_sha256(const char* path, long long data_offset, long long data_len, char* hex65) {
  FILE* f = fopen(path, "rb");
  MLF_REQUIRE(f != nullptr, "cannot open %s: %s", path, strerror(errno));
  fseek(f, (long)data_offset, SEEK_SET);
  Sha256 s;
  std::vector<uint8_t> buf(1 << 20);
  long long left = data_len;
  while (left > 0) {
    const size_t want = left < (long long)buf.size() ? (size_t)left : buf.size();
    const size_t n = fread(buf.data(), 1, want, f);
    if (n == 0) break;
    s.update(buf.data(), n);
    left -= n;
  }
  fclose(f);
  MLF_REQUIRE(left == 0, "payload of %s shorter than its header says", path);
  s.hex(hex65);
  return 0;
}
