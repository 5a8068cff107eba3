// SSD tier of the tiered tensor store: the reference's spill-file format
// `[ndim u32 LE][dims u64 LE ...][f32 LE data]` (rust-nn src/offload.rs:127-180).
// Reads land directly in the caller's buffer (a pinned host allocation that the device then pulls
// with one async copy), writes go through a temporary file + rename so a crash never leaves a torn spill.
#include <cerrno>
#include <cstdint>
#include <cstdio>
#include <cstring>
#include <fcntl.h>
#include <string>
#include <sys/stat.h>
#include <unistd.h>
#include <vector>

namespace {
bool write_all(int fd, const void* p, size_t n) {
  const char* c = (const char*)p;
  while (n) {
    ssize_t w = ::write(fd, c, n);
    if (w < 0) { if (errno == EINTR) continue; return false; }
    c += w; n -= (size_t)w;
  }
  return true;
}
bool read_all(int fd, void* p, size_t n) {
  char* c = (char*)p;
  while (n) {
    ssize_t r = ::read(fd, c, n);
    if (r < 0) { if (errno == EINTR) continue; return false; }
    if (r == 0) return false;
    c += r; n -= (size_t)r;
  }
  return true;
}
}  // namespace

extern "C" {

// returns bytes written, or -errno
long long b200_ssd_write(const char* path, const long long* shape, int ndim, const float* data, long long numel) {
  const std::string tmp = std::string(path) + ".tmp";
  int fd = ::open(tmp.c_str(), O_WRONLY | O_CREAT | O_TRUNC, 0600);
  if (fd < 0) return -errno;
  std::vector<uint8_t> hdr(4 + (size_t)ndim * 8);
  const uint32_t nd = (uint32_t)ndim;
  memcpy(hdr.data(), &nd, 4);
  for (int i = 0; i < ndim; ++i) { const uint64_t d = (uint64_t)shape[i]; memcpy(hdr.data() + 4 + 8 * i, &d, 8); }
  bool ok = write_all(fd, hdr.data(), hdr.size()) && write_all(fd, data, (size_t)numel * 4);
  const int e = errno;
  ::close(fd);
  if (!ok) { ::unlink(tmp.c_str()); return -e; }
  if (::rename(tmp.c_str(), path) != 0) { const int e2 = errno; ::unlink(tmp.c_str()); return -e2; }
  return (long long)hdr.size() + numel * 4;
}

// reads the header: fills shape (up to cap dims); returns ndim, or -1 (too short / unreadable)
int b200_ssd_header(const char* path, long long* shape, int cap, long long* numel_out) {
  int fd = ::open(path, O_RDONLY);
  if (fd < 0) return -1;
  uint32_t nd = 0;
  if (!read_all(fd, &nd, 4) || nd > 64) { ::close(fd); return -1; }
  long long numel = 1;
  for (uint32_t i = 0; i < nd; ++i) {
    uint64_t d;
    if (!read_all(fd, &d, 8)) { ::close(fd); return -1; }
    if ((int)i < cap) shape[i] = (long long)d;
    numel *= (long long)d;
  }
  struct stat st;
  if (fstat(fd, &st) != 0) { ::close(fd); return -1; }
  ::close(fd);
  const long long payload = (long long)st.st_size - 4 - 8LL * nd;
  if (payload < numel * 4) return -1;
  *numel_out = numel;
  return (int)nd;
}

// reads `numel` floats into `out` (skipping the header); returns 0 or -1
int b200_ssd_read(const char* path, float* out, long long numel) {
  int fd = ::open(path, O_RDONLY);
  if (fd < 0) return -1;
  uint32_t nd = 0;
  bool ok = read_all(fd, &nd, 4) && nd <= 64 && lseek(fd, 4 + 8LL * nd, SEEK_SET) >= 0 && read_all(fd, out, (size_t)numel * 4);
  ::close(fd);
  return ok ? 0 : -1;
}

}  // extern "C"
