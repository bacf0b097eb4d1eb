// Weight files on the host: a safetensors reader (memory-mapped, zero-copy views), the per-rank prepared
// file (writer + parallel pread loader with digests), and a 64-bit content digest.
//
// Reference behaviour: crates/sparkflash-weights/src/safetensors (header = u64 length + JSON table of
// dtype/shape/data_offsets), crates/sparkflash-weights/src/rank_file.rs:15-37 and
// crates/sparkflash-device/src/converted.rs:15-42 (one file per rank holding every tensor in its final device
// layout, a digest per tensor and one for the file, loaded with large parallel reads).
//
// Rank file layout (little endian):
//   [0,8)    magic "SFBRANK1"
//   payloads, each starting on a 4096-byte boundary
//   table    JSON: {"meta": <caller's JSON>, "tensors": [{"name","dtype","shape","offset","nbytes","digest"}]}
//   footer   u64 table_offset, u64 table_bytes, u64 table_digest, magic "SFBRANKE"
#include <fcntl.h>
#include <stdint.h>
#include <stdio.h>
#include <stdlib.h>
#include <string.h>
#include <sys/mman.h>
#include <sys/stat.h>
#include <unistd.h>

#include <atomic>
#include <string>
#include <thread>
#include <vector>

namespace {

// ---- digest: the XXH64 algorithm (public specification), seed 0 ------------------------------------------------
const uint64_t P1 = 11400714785074694791ull, P2 = 14029467366897019727ull, P3 = 1609587929392839161ull,
               P4 = 9650029242287828579ull, P5 = 2870177450012600261ull;
inline uint64_t rotl(uint64_t x, int r) { return (x << r) | (x >> (64 - r)); }
inline uint64_t rd64(const uint8_t* p) { uint64_t v; memcpy(&v, p, 8); return v; }
inline uint32_t rd32(const uint8_t* p) { uint32_t v; memcpy(&v, p, 4); return v; }
inline uint64_t round1(uint64_t acc, uint64_t in) { return rotl(acc + in * P2, 31) * P1; }
inline uint64_t merge(uint64_t acc, uint64_t v) { return (acc ^ round1(0, v)) * P1 + P4; }

uint64_t digest64(const void* data, size_t len) {
  const uint8_t* p = (const uint8_t*)data;
  const uint8_t* end = p + len;
  uint64_t h;
  if (len >= 32) {
    uint64_t v1 = P1 + P2, v2 = P2, v3 = 0, v4 = 0 - P1;
    const uint8_t* lim = end - 32;
    do {
      v1 = round1(v1, rd64(p)); v2 = round1(v2, rd64(p + 8)); v3 = round1(v3, rd64(p + 16)); v4 = round1(v4, rd64(p + 24));
      p += 32;
    } while (p <= lim);
    h = rotl(v1, 1) + rotl(v2, 7) + rotl(v3, 12) + rotl(v4, 18);
    h = merge(h, v1); h = merge(h, v2); h = merge(h, v3); h = merge(h, v4);
  } else {
    h = P5;
  }
  h += (uint64_t)len;
  while (p + 8 <= end) { h ^= round1(0, rd64(p)); h = rotl(h, 27) * P1 + P4; p += 8; }
  if (p + 4 <= end) { h ^= (uint64_t)rd32(p) * P1; h = rotl(h, 23) * P2 + P3; p += 4; }
  while (p < end) { h ^= (*p) * P5; h = rotl(h, 11) * P1; ++p; }
  h ^= h >> 33; h *= P2; h ^= h >> 29; h *= P3; h ^= h >> 32;
  return h;
}

// ---- a small JSON reader: enough for the two tables ----------------------------------------------------------------
struct J {
  const char* p; const char* e; bool ok = true;
  void ws() { while (p < e && (*p == ' ' || *p == '\n' || *p == '\t' || *p == '\r')) ++p; }
  bool eat(char c) { ws(); if (p < e && *p == c) { ++p; return true; } return false; }
  std::string str() {
    std::string s; ws();
    if (p >= e || *p != '"') { ok = false; return s; }
    ++p;
    while (p < e && *p != '"') {
      if (*p == '\\' && p + 1 < e) {
        ++p;
        switch (*p) { case 'n': s += '\n'; break; case 't': s += '\t'; break; case 'u': s += '?'; p += 4; break; default: s += *p; }
        ++p;
      } else s += *p++;
    }
    if (p < e) ++p; else ok = false;
    return s;
  }
  int64_t num() { ws(); char* q; long long v = strtoll(p, &q, 10); if (q == p) ok = false; p = q; return v; }
  void skip() {   // any value
    ws();
    if (p >= e) { ok = false; return; }
    if (*p == '"') { str(); return; }
    if (*p == '{' || *p == '[') {
      char open = *p, close = open == '{' ? '}' : ']';
      ++p;
      if (eat(close)) return;
      do { if (open == '{') { str(); if (!eat(':')) { ok = false; return; } } skip(); } while (ok && eat(','));
      if (!eat(close)) ok = false;
      return;
    }
    while (p < e && *p != ',' && *p != '}' && *p != ']') ++p;
  }
  std::string raw_value() { ws(); const char* s = p; skip(); return std::string(s, p - s); }
};

struct Entry { std::string name, dtype; std::vector<int64_t> shape; uint64_t offset = 0, nbytes = 0, digest = 0; };

struct Mapped {
  int fd = -1; uint8_t* base = nullptr; size_t size = 0;
  bool open(const char* path) {
    fd = ::open(path, O_RDONLY);
    if (fd < 0) return false;
    struct stat st; if (fstat(fd, &st)) return false;
    size = (size_t)st.st_size;
    base = (uint8_t*)mmap(nullptr, size, PROT_READ, MAP_PRIVATE, fd, 0);
    return base != MAP_FAILED;
  }
  ~Mapped() { if (base && base != MAP_FAILED) munmap(base, size); if (fd >= 0) close(fd); }
};

struct SafeTensors { Mapped m; std::vector<Entry> t; uint64_t data_start = 0; std::string meta; };

bool parse_entry_fields(J& j, Entry& en, bool st_style) {
  if (!j.eat('{')) return false;
  if (j.eat('}')) return true;
  do {
    std::string k = j.str();
    if (!j.eat(':')) return false;
    if (k == "dtype") en.dtype = j.str();
    else if (k == "name") en.name = j.str();
    else if (k == "shape") {
      if (!j.eat('[')) return false;
      if (!j.eat(']')) { do en.shape.push_back(j.num()); while (j.eat(',')); if (!j.eat(']')) return false; }
    } else if (k == "data_offsets" && st_style) {
      if (!j.eat('[')) return false;
      int64_t a = j.num(); if (!j.eat(',')) return false; int64_t b = j.num(); if (!j.eat(']')) return false;
      if (a < 0 || b < a) return false;            // reversed or negative range: never wraps into a huge length
      en.offset = (uint64_t)a; en.nbytes = (uint64_t)(b - a);
    } else if (k == "offset") { int64_t v = j.num(); if (v < 0) return false; en.offset = (uint64_t)v; }
    else if (k == "nbytes") { int64_t v = j.num(); if (v < 0) return false; en.nbytes = (uint64_t)v; }
    else if (k == "digest") { std::string d = j.str(); en.digest = strtoull(d.c_str(), nullptr, 16); }
    else j.skip();
  } while (j.ok && j.eat(','));
  return j.eat('}') && j.ok;
}

struct RankWriter { FILE* f = nullptr; uint64_t pos = 0; std::vector<Entry> t; };
struct RankReader { int fd = -1; std::vector<Entry> t; std::string meta; uint64_t file_size = 0; };

void json_escape(const std::string& s, std::string& out) {
  for (char c : s) { if (c == '"' || c == '\\') out += '\\'; out += c; }
}

thread_local std::string g_err;

// [offset, offset + nbytes) inside a region of `size` bytes, compared without overflow
bool range_inside(uint64_t offset, uint64_t nbytes, uint64_t size) { return offset <= size && nbytes <= size - offset; }

// bits per element of a safetensors / rank-file dtype (0 = unknown: the size check is skipped)
int dtype_bits(const std::string& d) {
  if (d == "F64" || d == "I64" || d == "U64") return 64;
  if (d == "F32" || d == "I32" || d == "U32") return 32;
  if (d == "F16" || d == "BF16" || d == "I16" || d == "U16") return 16;
  if (d == "F8_E4M3" || d == "F8_E5M2" || d == "F8_E8M0" || d == "I8" || d == "U8" || d == "BOOL") return 8;
  if (d == "F4") return 4;
  return 0;
}

// prod(shape) * element size == nbytes (packed 4-bit types count two elements per byte)
bool shape_matches(const Entry& en) {
  const int bits = dtype_bits(en.dtype);
  if (!bits) return true;
  unsigned __int128 n = 1;
  for (int64_t s : en.shape) {
    if (s < 0) return false;
    n *= (unsigned __int128)s;
    if (n > ((unsigned __int128)1 << 70)) return false;
  }
  const unsigned __int128 total_bits = n * (unsigned)bits;
  return total_bits == (unsigned __int128)en.nbytes * 8 || (bits == 4 && ((total_bits + 4) / 8 == en.nbytes || n == en.nbytes));
}

}  // namespace

extern "C" {

const char* sfb_weights_last_error() { return g_err.c_str(); }
uint64_t sfb_digest64(const void* p, uint64_t n) { return digest64(p, (size_t)n); }

// ---- safetensors ---------------------------------------------------------------------------------------------------
void* sfb_st_open(const char* path) {
  SafeTensors* s = new SafeTensors();
  if (!s->m.open(path) || s->m.size < 8) { g_err = std::string("cannot map ") + path; delete s; return nullptr; }
  uint64_t hl = rd64(s->m.base);
  if (hl > s->m.size - 8) { g_err = "header length beyond the file"; delete s; return nullptr; }
  s->data_start = 8 + hl;
  J j{(const char*)s->m.base + 8, (const char*)s->m.base + 8 + hl};
  if (!j.eat('{')) { g_err = "header is not a JSON object"; delete s; return nullptr; }
  if (!j.eat('}')) {
    do {
      std::string name = j.str();
      if (!j.eat(':')) { j.ok = false; break; }
      if (name == "__metadata__") { s->meta = j.raw_value(); continue; }
      Entry en; en.name = name;
      if (!parse_entry_fields(j, en, true)) { j.ok = false; break; }
      if (!range_inside(en.offset, en.nbytes, s->m.size - s->data_start)) { g_err = "tensor " + name + " lies beyond the file"; delete s; return nullptr; }
      if (!shape_matches(en)) { g_err = "tensor " + name + ": shape and dtype do not give its byte length"; delete s; return nullptr; }
      s->t.push_back(en);
    } while (j.ok && j.eat(','));
  }
  if (!j.ok) { g_err = "malformed safetensors header"; delete s; return nullptr; }
  return s;
}
void sfb_st_close(void* h) { delete (SafeTensors*)h; }
int sfb_st_count(void* h) { return (int)((SafeTensors*)h)->t.size(); }
const char* sfb_st_name(void* h, int i) { return ((SafeTensors*)h)->t[i].name.c_str(); }
const char* sfb_st_dtype(void* h, int i) { return ((SafeTensors*)h)->t[i].dtype.c_str(); }
int sfb_st_shape(void* h, int i, int64_t* out8) {
  auto& sh = ((SafeTensors*)h)->t[i].shape;
  for (size_t k = 0; k < sh.size() && k < 8; ++k) out8[k] = sh[k];
  return (int)sh.size();
}
const void* sfb_st_data(void* h, int i, uint64_t* nbytes) {
  SafeTensors* s = (SafeTensors*)h;
  *nbytes = s->t[i].nbytes;
  return s->m.base + s->data_start + s->t[i].offset;
}

// ---- rank file: writer ------------------------------------------------------------------------------------------------
void* sfb_rank_writer_open(const char* path) {
  FILE* f = fopen(path, "wb");
  if (!f) { g_err = std::string("cannot create ") + path; return nullptr; }
  RankWriter* w = new RankWriter(); w->f = f;
  fwrite("SFBRANK1", 1, 8, f); w->pos = 8;
  return w;
}
int sfb_rank_writer_add(void* h, const char* name, const char* dtype, int ndim, const int64_t* shape, const void* data, uint64_t nbytes) {
  RankWriter* w = (RankWriter*)h;
  static const char zeros[4096] = {0};
  uint64_t pad = (4096 - w->pos % 4096) % 4096;
  if (pad && fwrite(zeros, 1, pad, w->f) != pad) { g_err = "short write"; return 1; }
  w->pos += pad;
  Entry en; en.name = name; en.dtype = dtype; en.shape.assign(shape, shape + ndim); en.offset = w->pos; en.nbytes = nbytes;
  en.digest = digest64(data, nbytes);
  if (nbytes && fwrite(data, 1, nbytes, w->f) != nbytes) { g_err = "short write"; return 1; }
  w->pos += nbytes;
  w->t.push_back(en);
  return 0;
}
int sfb_rank_writer_close(void* h, const char* meta_json) {
  RankWriter* w = (RankWriter*)h;
  std::string tb = "{\"meta\": "; tb += (meta_json && *meta_json) ? meta_json : "{}"; tb += ", \"tensors\": [";
  char buf[160];
  for (size_t i = 0; i < w->t.size(); ++i) {
    const Entry& e = w->t[i];
    if (i) tb += ", ";
    tb += "{\"name\": \""; json_escape(e.name, tb); tb += "\", \"dtype\": \"" + e.dtype + "\", \"shape\": [";
    for (size_t k = 0; k < e.shape.size(); ++k) { snprintf(buf, sizeof buf, "%s%lld", k ? ", " : "", (long long)e.shape[k]); tb += buf; }
    snprintf(buf, sizeof buf, "], \"offset\": %llu, \"nbytes\": %llu, \"digest\": \"%016llx\"}", (unsigned long long)e.offset,
             (unsigned long long)e.nbytes, (unsigned long long)e.digest);
    tb += buf;
  }
  tb += "]}";
  uint64_t off = w->pos, n = tb.size(), d = digest64(tb.data(), tb.size());
  int rc = 0;
  if (fwrite(tb.data(), 1, n, w->f) != n) rc = 1;
  fwrite(&off, 8, 1, w->f); fwrite(&n, 8, 1, w->f); fwrite(&d, 8, 1, w->f); fwrite("SFBRANKE", 1, 8, w->f);
  if (fclose(w->f)) rc = 1;
  if (rc) g_err = "short write";
  delete w;
  return rc;
}

// ---- rank file: reader ---------------------------------------------------------------------------------------------------
void* sfb_rank_open(const char* path) {
  int fd = ::open(path, O_RDONLY);
  if (fd < 0) { g_err = std::string("cannot open ") + path; return nullptr; }
  struct stat st; fstat(fd, &st);
  uint8_t foot[32], magic[8];
  if (st.st_size < 40 || pread(fd, magic, 8, 0) != 8 || memcmp(magic, "SFBRANK1", 8) ||
      pread(fd, foot, 32, st.st_size - 32) != 32 || memcmp(foot + 24, "SFBRANKE", 8)) {
    g_err = "not a rank file (magic or footer missing: truncated?)"; close(fd); return nullptr;
  }
  uint64_t off = rd64(foot), n = rd64(foot + 8), d = rd64(foot + 16);
  if (off + n + 32 != (uint64_t)st.st_size) { g_err = "table does not end at the footer"; close(fd); return nullptr; }
  std::string tb(n, '\0');
  if ((uint64_t)pread(fd, &tb[0], n, off) != n || digest64(tb.data(), n) != d) { g_err = "table digest mismatch"; close(fd); return nullptr; }
  RankReader* r = new RankReader(); r->fd = fd; r->file_size = st.st_size;
  J j{tb.data(), tb.data() + n};
  bool ok = j.eat('{');
  while (ok) {
    std::string k = j.str();
    if (!j.eat(':')) { ok = false; break; }
    if (k == "meta") r->meta = j.raw_value();
    else if (k == "tensors") {
      if (!j.eat('[')) { ok = false; break; }
      if (!j.eat(']')) {
        do { Entry en; if (!parse_entry_fields(j, en, false)) { ok = false; break; } r->t.push_back(en); } while (j.eat(','));
        if (ok && !j.eat(']')) ok = false;
      }
    } else j.skip();
    if (!j.eat(',')) break;
  }
  if (!ok || !j.ok) { g_err = "malformed table"; close(fd); delete r; return nullptr; }
  for (auto& e : r->t) if (!range_inside(e.offset, e.nbytes, off)) { g_err = "tensor " + e.name + " overlaps the table"; close(fd); delete r; return nullptr; }
  return r;
}
void sfb_rank_close(void* h) { RankReader* r = (RankReader*)h; if (r->fd >= 0) close(r->fd); delete r; }
int sfb_rank_count(void* h) { return (int)((RankReader*)h)->t.size(); }
const char* sfb_rank_meta(void* h) { return ((RankReader*)h)->meta.c_str(); }
const char* sfb_rank_name(void* h, int i) { return ((RankReader*)h)->t[i].name.c_str(); }
const char* sfb_rank_dtype(void* h, int i) { return ((RankReader*)h)->t[i].dtype.c_str(); }
int sfb_rank_shape(void* h, int i, int64_t* out8) {
  auto& sh = ((RankReader*)h)->t[i].shape;
  for (size_t k = 0; k < sh.size() && k < 8; ++k) out8[k] = sh[k];
  return (int)sh.size();
}
uint64_t sfb_rank_nbytes(void* h, int i) { return ((RankReader*)h)->t[i].nbytes; }

// Read tensors [first, first+count) into dst + dst_offsets[k] with `threads` workers issuing reads of at most
// 8 MiB; verify != 0 checks every digest.  Returns 0, or 1 + index of the first tensor that failed.
int sfb_rank_read(void* h, int first, int count, uint8_t* dst, const uint64_t* dst_offsets, int threads, int verify) {
  RankReader* r = (RankReader*)h;
  struct Job { uint64_t src, dst, n; };
  std::vector<Job> jobs;
  const uint64_t CH = 8ull << 20;
  for (int k = 0; k < count; ++k) {
    const Entry& e = r->t[first + k];
    for (uint64_t o = 0; o < e.nbytes; o += CH) jobs.push_back({e.offset + o, dst_offsets[k] + o, std::min(CH, e.nbytes - o)});
  }
  std::atomic<size_t> next{0};
  std::atomic<int> bad{0};
  auto work = [&]() {
    for (;;) {
      size_t i = next.fetch_add(1);
      if (i >= jobs.size()) return;
      uint64_t done = 0;
      while (done < jobs[i].n) {
        ssize_t got = pread(r->fd, dst + jobs[i].dst + done, jobs[i].n - done, jobs[i].src + done);
        if (got <= 0) { bad = 1; return; }
        done += (uint64_t)got;
      }
    }
  };
  threads = std::max(1, std::min(threads, 64));
  std::vector<std::thread> pool;
  for (int t = 1; t < threads; ++t) pool.emplace_back(work);
  work();
  for (auto& t : pool) t.join();
  if (bad) { g_err = "short read"; return 1 + first; }
  if (verify) {
    std::atomic<int> fail{-1};
    std::atomic<int> nk{0};
    auto chk = [&]() {
      for (;;) {
        int k = nk.fetch_add(1);
        if (k >= count) return;
        const Entry& e = r->t[first + k];
        if (digest64(dst + dst_offsets[k], e.nbytes) != e.digest) { int exp = -1; fail.compare_exchange_strong(exp, first + k); }
      }
    };
    std::vector<std::thread> p2;
    for (int t = 1; t < threads; ++t) p2.emplace_back(chk);
    chk();
    for (auto& t : p2) t.join();
    if (fail >= 0) { g_err = "digest mismatch in tensor " + r->t[fail].name; return 1 + fail; }
  }
  return 0;
}

}  // extern "C"
