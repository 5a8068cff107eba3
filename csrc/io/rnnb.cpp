// Checkpoint I/O in C++: the byte-exact `rnnb` v1 container and F32 safetensors export/import.
//
// rnnb v1 (rust-nn src/serialize.rs:3-16, 29-52):
//   "RNNB" | u32 version = 1 | u32 count | count x { u32 name_len | name | u32 ndim | u64 dims[ndim] |
//   u32 numel | f32 data[numel] }           (all little-endian)
// numel is a u32, so tensors above 2^32-1 elements are rejected rather than written wrongly.
// Files are written atomically (temp file + rename) and read through mmap.
#include <cerrno>
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

enum : int { IO_OK = 0, IO_BAD_MAGIC = 1, IO_BAD_VERSION = 2, IO_TRUNCATED = 3, IO_TOO_LARGE = 4, IO_BAD_ARG = 5,
             IO_SYS = 6, IO_BAD_JSON = 7, IO_NUMEL_MISMATCH = 8 };

inline void put_u32(uint8_t*& p, uint32_t v) { memcpy(p, &v, 4); p += 4; }
inline void put_u64(uint8_t*& p, uint64_t v) { memcpy(p, &v, 8); p += 8; }
inline bool get_u32(const uint8_t* b, int64_t len, int64_t& off, uint32_t& v) {
  if (off + 4 > len) return false;
  memcpy(&v, b + off, 4);
  off += 4;
  return true;
}
inline bool get_u64(const uint8_t* b, int64_t len, int64_t& off, uint64_t& v) {
  if (off + 8 > len) return false;
  memcpy(&v, b + off, 8);
  off += 8;
  return true;
}

}  // namespace

extern "C" {

// Size in bytes of the serialized container. Returns -1 if a tensor cannot be represented.
long long b200_rnnb_size(int count, const int* name_lens, const int* ndims, const long long* numels) {
  long long total = 12;
  for (int i = 0; i < count; ++i) {
    if (numels[i] < 0 || numels[i] > 0xFFFFFFFFLL) return -1;
    total += 4 + name_lens[i] + 4 + 8LL * ndims[i] + 4 + 4LL * numels[i];
  }
  return total;
}

// dims_flat holds the dims of all tensors back to back. `data[i]` points at numel f32 values.
int b200_rnnb_serialize(int count, const char* const* names, const int* name_lens, const int* ndims,
                        const long long* dims_flat, const long long* numels, const float* const* data,
                        unsigned char* out, long long out_cap) {
  long long need = b200_rnnb_size(count, name_lens, ndims, numels);
  if (need < 0) return IO_TOO_LARGE;
  if (need > out_cap) return IO_BAD_ARG;
  uint8_t* p = out;
  memcpy(p, "RNNB", 4); p += 4;
  put_u32(p, 1);
  put_u32(p, (uint32_t)count);
  const long long* d = dims_flat;
  for (int i = 0; i < count; ++i) {
    put_u32(p, (uint32_t)name_lens[i]);
    memcpy(p, names[i], name_lens[i]); p += name_lens[i];
    put_u32(p, (uint32_t)ndims[i]);
    long long prod = 1;
    for (int k = 0; k < ndims[i]; ++k) { put_u64(p, (uint64_t)d[k]); prod *= d[k]; }
    d += ndims[i];
    if (prod != numels[i]) return IO_NUMEL_MISMATCH;
    put_u32(p, (uint32_t)numels[i]);
    memcpy(p, data[i], 4ULL * numels[i]); p += 4ULL * numels[i];
  }
  return IO_OK;
}

// Validates magic/version and returns the tensor count.
int b200_rnnb_header(const unsigned char* buf, long long len, int* count) {
  if (len < 12) return len >= 4 && memcmp(buf, "RNNB", 4) != 0 ? IO_BAD_MAGIC : IO_TRUNCATED;
  if (memcmp(buf, "RNNB", 4) != 0) return IO_BAD_MAGIC;
  uint32_t ver, cnt; memcpy(&ver, buf + 4, 4); memcpy(&cnt, buf + 8, 4);
  if (ver != 1) return IO_BAD_VERSION;
  *count = (int)cnt;
  return IO_OK;
}

// Index of every tensor: byte offsets of name / dims / data inside `buf`.
int b200_rnnb_index(const unsigned char* buf, long long len, int count, long long* name_off, int* name_len,
                    int* ndim, long long* dims_off, long long* numel, long long* data_off) {
  int64_t off = 12;
  for (int i = 0; i < count; ++i) {
    uint32_t nl, nd, ne;
    if (!get_u32(buf, len, off, nl)) return IO_TRUNCATED;
    if (off + nl > len) return IO_TRUNCATED;
    name_off[i] = off; name_len[i] = (int)nl; off += nl;
    if (!get_u32(buf, len, off, nd)) return IO_TRUNCATED;
    if (nd > 64) return IO_BAD_ARG;
    ndim[i] = (int)nd; dims_off[i] = off;
    uint64_t prod = 1;
    for (uint32_t k = 0; k < nd; ++k) { uint64_t dv; if (!get_u64(buf, len, off, dv)) return IO_TRUNCATED; prod *= dv; }
    if (!get_u32(buf, len, off, ne)) return IO_TRUNCATED;
    if (prod != ne) return IO_NUMEL_MISMATCH;
    if (off + 4LL * ne > len) return IO_TRUNCATED;
    numel[i] = ne; data_off[i] = off; off += 4LL * ne;
  }
  return IO_OK;
}

// ------------------------------------------------------------------ files
int b200_file_write_atomic(const char* path, const unsigned char* buf, long long len) {
  std::string tmp = std::string(path) + ".tmp." + std::to_string((long long)getpid());
  int fd = open(tmp.c_str(), O_WRONLY | O_CREAT | O_TRUNC, 0644);
  if (fd < 0) return IO_SYS;
  long long done = 0;
  while (done < len) {
    ssize_t w = write(fd, buf + done, (size_t)std::min<long long>(len - done, 1LL << 30));
    if (w < 0) { if (errno == EINTR) continue; close(fd); unlink(tmp.c_str()); return IO_SYS; }
    done += w;
  }
  if (fsync(fd) != 0) { close(fd); unlink(tmp.c_str()); return IO_SYS; }
  close(fd);
  if (rename(tmp.c_str(), path) != 0) { unlink(tmp.c_str()); return IO_SYS; }
  return IO_OK;
}

long long b200_file_size(const char* path) {
  struct stat st;
  if (stat(path, &st) != 0) return -1;
  return (long long)st.st_size;
}

// Reads the whole file into `out` (capacity `cap`) through mmap. Returns bytes read or -1.
long long b200_file_read(const char* path, unsigned char* out, long long cap) {
  int fd = open(path, O_RDONLY);
  if (fd < 0) return -1;
  struct stat st;
  if (fstat(fd, &st) != 0) { close(fd); return -1; }
  long long len = st.st_size;
  if (len > cap) { close(fd); return -1; }
  if (len == 0) { close(fd); return 0; }
  void* m = mmap(nullptr, (size_t)len, PROT_READ, MAP_PRIVATE, fd, 0);
  close(fd);
  if (m == MAP_FAILED) return -1;
  memcpy(out, m, (size_t)len);
  munmap(m, (size_t)len);
  return len;
}

// ------------------------------------------------------------------ safetensors (F32 only)
// Layout: u64 header_len | JSON header | raw data. Header entries:
//   "name": {"dtype":"F32","shape":[...],"data_offsets":[begin,end]}
static void json_escape(std::string& out, const char* s, int n) {
  for (int i = 0; i < n; ++i) {
    unsigned char c = (unsigned char)s[i];
    if (c == '"' || c == '\\') { out.push_back('\\'); out.push_back((char)c); }
    else if (c < 0x20) { char b[8]; snprintf(b, sizeof b, "\\u%04x", c); out += b; }
    else out.push_back((char)c);
  }
}

static std::string st_header(int count, const char* const* names, const int* name_lens, const int* ndims,
                             const long long* dims_flat, const long long* numels) {
  std::string h = "{";
  const long long* d = dims_flat;
  long long off = 0;
  for (int i = 0; i < count; ++i) {
    if (i) h += ",";
    h += "\""; json_escape(h, names[i], name_lens[i]); h += "\":{\"dtype\":\"F32\",\"shape\":[";
    for (int k = 0; k < ndims[i]; ++k) { if (k) h += ","; h += std::to_string(d[k]); }
    d += ndims[i];
    h += "],\"data_offsets\":[" + std::to_string(off) + "," + std::to_string(off + 4 * numels[i]) + "]}";
    off += 4 * numels[i];
  }
  h += "}";
  while ((h.size() + 8) % 8 != 0) h.push_back(' ');
  return h;
}

long long b200_safetensors_size(int count, const char* const* names, const int* name_lens, const int* ndims,
                                const long long* dims_flat, const long long* numels) {
  std::string h = st_header(count, names, name_lens, ndims, dims_flat, numels);
  long long total = 8 + (long long)h.size();
  for (int i = 0; i < count; ++i) total += 4 * numels[i];
  return total;
}

int b200_safetensors_export(int count, const char* const* names, const int* name_lens, const int* ndims,
                            const long long* dims_flat, const long long* numels, const float* const* data,
                            unsigned char* out, long long out_cap) {
  std::string h = st_header(count, names, name_lens, ndims, dims_flat, numels);
  long long total = 8 + (long long)h.size();
  for (int i = 0; i < count; ++i) total += 4 * numels[i];
  if (total > out_cap) return IO_BAD_ARG;
  uint8_t* p = out;
  put_u64(p, (uint64_t)h.size());
  memcpy(p, h.data(), h.size()); p += h.size();
  for (int i = 0; i < count; ++i) { memcpy(p, data[i], 4ULL * numels[i]); p += 4ULL * numels[i]; }
  return IO_OK;
}

// Minimal JSON walk over the (flat, two-level) safetensors header. Fills up to `cap` entries; returns the
// number of tensors found (entries named "__metadata__" are skipped), or a negative error code.
int b200_safetensors_index(const unsigned char* buf, long long len, int cap, long long* name_off, int* name_len,
                           int* ndim, long long* dims /* cap x 8 */, long long* data_begin, long long* data_end,
                           long long* data_base) {
  if (len < 8) return -IO_TRUNCATED;
  uint64_t hl; memcpy(&hl, buf, 8);
  if (8 + (long long)hl > len) return -IO_TRUNCATED;
  *data_base = 8 + (long long)hl;
  const char* s = (const char*)buf + 8;
  long long n = (long long)hl, i = 0;
  auto skip_ws = [&]() { while (i < n && (s[i] == ' ' || s[i] == '\n' || s[i] == '\t' || s[i] == '\r')) ++i; };
  auto parse_string = [&](long long& b, long long& e) -> bool {
    skip_ws();
    if (i >= n || s[i] != '"') return false;
    ++i; b = i;
    while (i < n && s[i] != '"') { if (s[i] == '\\') ++i; ++i; }
    if (i >= n) return false;
    e = i; ++i;
    return true;
  };
  // skip any JSON value (used for __metadata__ and unknown keys)
  auto skip_value = [&]() -> bool {
    skip_ws(); if (i >= n) return false;
    int depth = 0; bool in_str = false;
    for (; i < n; ++i) {
      char c = s[i];
      if (in_str) { if (c == '\\') ++i; else if (c == '"') in_str = false; continue; }
      if (c == '"') in_str = true;
      else if (c == '{' || c == '[') ++depth;
      else if (c == '}' || c == ']') { if (depth == 0) return true; --depth; if (depth == 0) { ++i; return true; } }
      else if (c == ',' && depth == 0) return true;
    }
    return true;
  };
  skip_ws(); if (i >= n || s[i] != '{') return -IO_BAD_JSON; ++i;
  int found = 0;
  while (true) {
    skip_ws(); if (i < n && s[i] == '}') break;
    long long kb, ke; if (!parse_string(kb, ke)) return -IO_BAD_JSON;
    skip_ws(); if (i >= n || s[i] != ':') return -IO_BAD_JSON; ++i;
    bool meta = (ke - kb == 12 && memcmp(s + kb, "__metadata__", 12) == 0);
    if (meta) { if (!skip_value()) return -IO_BAD_JSON; }
    else {
      skip_ws(); if (i >= n || s[i] != '{') return -IO_BAD_JSON; ++i;
      int nd = 0; long long dd[8] = {0}; long long db = -1, de = -1; bool f32 = false;
      while (true) {
        skip_ws(); if (i < n && s[i] == '}') { ++i; break; }
        long long fb, fe; if (!parse_string(fb, fe)) return -IO_BAD_JSON;
        skip_ws(); if (i >= n || s[i] != ':') return -IO_BAD_JSON; ++i;
        std::string key(s + fb, s + fe);
        if (key == "dtype") { long long vb, ve; if (!parse_string(vb, ve)) return -IO_BAD_JSON; f32 = (ve - vb == 3 && memcmp(s + vb, "F32", 3) == 0); }
        else if (key == "shape" || key == "data_offsets") {
          skip_ws(); if (i >= n || s[i] != '[') return -IO_BAD_JSON; ++i;
          std::vector<long long> vals;
          while (true) { skip_ws(); if (i < n && s[i] == ']') { ++i; break; }
            char* endp; long long v = strtoll(s + i, &endp, 10); if (endp == s + i) return -IO_BAD_JSON; i = endp - s; vals.push_back(v);
            skip_ws(); if (i < n && s[i] == ',') ++i; }
          if (key == "shape") { nd = (int)vals.size(); if (nd > 8) return -IO_BAD_ARG; for (int k = 0; k < nd; ++k) dd[k] = vals[k]; }
          else { if (vals.size() != 2) return -IO_BAD_JSON; db = vals[0]; de = vals[1]; }
        } else { if (!skip_value()) return -IO_BAD_JSON; }
        skip_ws(); if (i < n && s[i] == ',') ++i;
      }
      if (!f32 || db < 0 || de < db || *data_base + de > len) return -IO_BAD_ARG;
      if (found < cap) {
        name_off[found] = 8 + kb; name_len[found] = (int)(ke - kb); ndim[found] = nd;
        for (int k = 0; k < 8; ++k) dims[found * 8 + k] = dd[k];
        data_begin[found] = db; data_end[found] = de;
      }
      ++found;
    }
    skip_ws(); if (i < n && s[i] == ',') ++i;
  }
  return found;
}

}  // extern "C"
