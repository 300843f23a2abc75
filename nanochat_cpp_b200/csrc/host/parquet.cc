// Minimal Parquet reader for text corpora: one BYTE_ARRAY column (REQUIRED or OPTIONAL, not nested),
// DATA_PAGE v1, PLAIN encoding, RLE/bit-packed definition levels, UNCOMPRESSED pages, and ZSTD pages when
// libzstd can be loaded at run time (dlopen: the library is not a build dependency). Same scope as the
// reference reader (src/parquet/reader.cc, format.cc, thrift.cc, levels.cc), written against the public
// Parquet and Thrift-compact specifications.
#include <dlfcn.h>

#include <cstring>
#include <fstream>

#include "core.h"

namespace ncb {

namespace {

// ---- Thrift compact protocol -------------------------------------------------------------------
class Thrift {
 public:
  Thrift(const std::uint8_t* p, std::size_t n) : p_(p), end_(p + n) {}
  bool ok() const { return ok_; }
  const std::uint8_t* pos() const { return p_; }

  std::uint64_t Varint() {
    std::uint64_t v = 0;
    int shift = 0;
    while (p_ < end_) {
      const std::uint8_t b = *p_++;
      v |= static_cast<std::uint64_t>(b & 0x7f) << shift;
      if (!(b & 0x80)) return v;
      shift += 7;
      if (shift > 63) break;
    }
    ok_ = false;
    return 0;
  }
  std::int64_t Zigzag() {
    const std::uint64_t v = Varint();
    return static_cast<std::int64_t>(v >> 1) ^ -static_cast<std::int64_t>(v & 1);
  }
  std::string Binary() {
    const std::uint64_t n = Varint();
    if (!ok_ || n > static_cast<std::uint64_t>(end_ - p_)) {
      ok_ = false;
      return {};
    }
    std::string s(reinterpret_cast<const char*>(p_), n);
    p_ += n;
    return s;
  }
  // Reads a field header; returns false at STOP. `type` is the compact type id.
  bool Field(int* id, int* type, int* last_id) {
    if (p_ >= end_) {
      ok_ = false;
      return false;
    }
    const std::uint8_t b = *p_++;
    if (b == 0) return false;
    *type = b & 0x0f;
    const int delta = b >> 4;
    *id = delta ? *last_id + delta : static_cast<int>(Zigzag());
    *last_id = *id;
    return ok_;
  }
  void ListHeader(int* elem_type, std::uint32_t* size) {
    if (p_ >= end_) {
      ok_ = false;
      return;
    }
    const std::uint8_t b = *p_++;
    *elem_type = b & 0x0f;
    *size = b >> 4;
    if (*size == 15) *size = static_cast<std::uint32_t>(Varint());
  }
  void Skip(int type) {
    switch (type) {
      case 1: case 2: return;                      // bool true / false (value in the header)
      case 3: if (p_ < end_) ++p_; else ok_ = false; return;  // byte
      case 4: case 5: case 6: Zigzag(); return;    // i16 / i32 / i64
      case 7: if (end_ - p_ >= 8) p_ += 8; else ok_ = false; return;  // double
      case 8: Binary(); return;
      case 9: case 10: {                           // list / set
        int et = 0;
        std::uint32_t n = 0;
        ListHeader(&et, &n);
        for (std::uint32_t i = 0; i < n && ok_; ++i) Skip(et == 1 || et == 2 ? 3 : et);
        return;
      }
      case 11: {                                   // map
        const std::uint64_t n = Varint();
        if (n == 0) return;
        if (p_ >= end_) { ok_ = false; return; }
        const std::uint8_t kv = *p_++;
        for (std::uint64_t i = 0; i < n && ok_; ++i) {
          Skip(kv >> 4);
          Skip(kv & 0x0f);
        }
        return;
      }
      case 12: {                                   // struct
        int id = 0, t = 0, last = 0;
        while (Field(&id, &t, &last)) Skip(t);
        return;
      }
      default: ok_ = false;
    }
  }

 private:
  const std::uint8_t* p_;
  const std::uint8_t* end_;
  bool ok_ = true;
};

struct SchemaElement {
  std::string name;
  int type = -1, repetition = 0, num_children = 0;
};
struct ColumnChunk {
  std::vector<std::string> path;
  int type = -1, codec = 0;
  std::int64_t num_values = 0, data_page_offset = -1, dict_page_offset = -1, total_compressed = 0;
};

bool Fail(std::string* error, const std::string& msg) {
  if (error != nullptr) *error = msg;
  return false;
}

void ParseColumnMeta(Thrift& t, ColumnChunk* c) {
  int id = 0, ty = 0, last = 0;
  while (t.Field(&id, &ty, &last)) {
    switch (id) {
      case 1: c->type = static_cast<int>(t.Zigzag()); break;
      case 3: {
        int et = 0;
        std::uint32_t n = 0;
        t.ListHeader(&et, &n);
        for (std::uint32_t i = 0; i < n && t.ok(); ++i) c->path.push_back(t.Binary());
        break;
      }
      case 4: c->codec = static_cast<int>(t.Zigzag()); break;
      case 5: c->num_values = t.Zigzag(); break;
      case 7: c->total_compressed = t.Zigzag(); break;
      case 9: c->data_page_offset = t.Zigzag(); break;
      case 11: c->dict_page_offset = t.Zigzag(); break;
      default: t.Skip(ty);
    }
  }
}

using ZstdDecompressFn = std::size_t (*)(void*, std::size_t, const void*, std::size_t);
using ZstdIsErrorFn = unsigned (*)(std::size_t);
bool ZstdDecompress(const std::uint8_t* src, std::size_t n, std::vector<std::uint8_t>* dst, std::string* error) {
  static ZstdDecompressFn fn = nullptr;
  static ZstdIsErrorFn is_err = nullptr;
  static bool tried = false;
  if (!tried) {
    tried = true;
    for (const char* name : {"libzstd.so.1", "libzstd.so"}) {
      if (void* h = dlopen(name, RTLD_NOW | RTLD_LOCAL)) {
        fn = reinterpret_cast<ZstdDecompressFn>(dlsym(h, "ZSTD_decompress"));
        is_err = reinterpret_cast<ZstdIsErrorFn>(dlsym(h, "ZSTD_isError"));
        if (fn != nullptr && is_err != nullptr) break;
      }
    }
  }
  if (fn == nullptr || is_err == nullptr) return Fail(error, "parquet page is ZSTD-compressed and libzstd is not available");
  const std::size_t got = fn(dst->data(), dst->size(), src, n);
  if (is_err(got) || got != dst->size()) return Fail(error, "parquet: ZSTD decompression failed");
  return true;
}

// RLE / bit-packed hybrid, bit width 1 (definition levels of a flat OPTIONAL column).
bool DecodeLevels(const std::uint8_t* p, std::size_t n, std::int64_t count, std::vector<std::uint8_t>* out) {
  Thrift v(p, n);
  out->clear();
  while (static_cast<std::int64_t>(out->size()) < count && v.ok() && v.pos() < p + n) {
    const std::uint64_t header = v.Varint();
    if (header & 1) {  // bit-packed groups of 8 values
      const std::uint64_t groups = header >> 1;
      const std::uint8_t* q = v.pos();
      if (groups > static_cast<std::uint64_t>(p + n - q)) return false;
      for (std::uint64_t g = 0; g < groups; ++g)
        for (int b = 0; b < 8; ++b) out->push_back((q[g] >> b) & 1);
      v = Thrift(q + groups, static_cast<std::size_t>(p + n - (q + groups)));
    } else {  // run of one value, stored in ceil(width / 8) = 1 byte
      const std::uint64_t run = header >> 1;
      const std::uint8_t* q = v.pos();
      if (q >= p + n) return false;
      out->insert(out->end(), run, *q & 1);
      v = Thrift(q + 1, static_cast<std::size_t>(p + n - (q + 1)));
    }
  }
  out->resize(static_cast<std::size_t>(count), 0);
  return true;
}

}  // namespace

bool ReadParquetStrings(const std::string& path, const std::string& column, std::vector<std::string>* out,
                        std::string* error) {
  std::ifstream f(path, std::ios::binary);
  if (!f) return Fail(error, "cannot open " + path);
  std::vector<std::uint8_t> file((std::istreambuf_iterator<char>(f)), std::istreambuf_iterator<char>());
  if (file.size() < 12 || std::memcmp(file.data(), "PAR1", 4) != 0 ||
      std::memcmp(file.data() + file.size() - 4, "PAR1", 4) != 0)
    return Fail(error, "not a parquet file: " + path);
  std::uint32_t footer_len = 0;
  std::memcpy(&footer_len, file.data() + file.size() - 8, 4);
  if (footer_len + 12ull > file.size()) return Fail(error, "parquet footer length is invalid: " + path);
  Thrift t(file.data() + file.size() - 8 - footer_len, footer_len);
  std::vector<SchemaElement> schema;
  std::vector<ColumnChunk> chunks;
  int id = 0, ty = 0, last = 0;
  while (t.Field(&id, &ty, &last)) {
    if (id == 2) {  // schema
      int et = 0;
      std::uint32_t n = 0;
      t.ListHeader(&et, &n);
      for (std::uint32_t i = 0; i < n && t.ok(); ++i) {
        SchemaElement e;
        int fid = 0, fty = 0, flast = 0;
        while (t.Field(&fid, &fty, &flast)) {
          if (fid == 1) e.type = static_cast<int>(t.Zigzag());
          else if (fid == 3) e.repetition = static_cast<int>(t.Zigzag());
          else if (fid == 4) e.name = t.Binary();
          else if (fid == 5) e.num_children = static_cast<int>(t.Zigzag());
          else t.Skip(fty);
        }
        schema.push_back(std::move(e));
      }
    } else if (id == 4) {  // row groups
      int et = 0;
      std::uint32_t n = 0;
      t.ListHeader(&et, &n);
      for (std::uint32_t i = 0; i < n && t.ok(); ++i) {
        int gid = 0, gty = 0, glast = 0;
        while (t.Field(&gid, &gty, &glast)) {
          if (gid == 1) {  // columns
            int cet = 0;
            std::uint32_t cn = 0;
            t.ListHeader(&cet, &cn);
            for (std::uint32_t c = 0; c < cn && t.ok(); ++c) {
              ColumnChunk chunk;
              int cid = 0, cty = 0, clast = 0;
              while (t.Field(&cid, &cty, &clast)) {
                if (cid == 3) ParseColumnMeta(t, &chunk);
                else t.Skip(cty);
              }
              chunks.push_back(std::move(chunk));
            }
          } else {
            t.Skip(gty);
          }
        }
      }
    } else {
      t.Skip(ty);
    }
  }
  if (!t.ok()) return Fail(error, "parquet footer is malformed: " + path);
  int repetition = -1;
  for (std::size_t i = 1; i < schema.size(); ++i)
    if (schema[i].name == column && schema[i].num_children == 0) repetition = schema[i].repetition;
  if (repetition < 0) return Fail(error, "parquet column '" + column + "' not found in " + path);
  if (repetition == 2) return Fail(error, "parquet column '" + column + "' is REPEATED, which is not supported");
  out->clear();
  for (const ColumnChunk& c : chunks) {
    if (c.path.size() != 1 || c.path[0] != column) continue;
    if (c.type != 6) return Fail(error, "parquet column '" + column + "' is not BYTE_ARRAY");
    if (c.codec != 0 && c.codec != 6) return Fail(error, "parquet codec is neither UNCOMPRESSED nor ZSTD");
    if (c.dict_page_offset > 0) return Fail(error, "parquet dictionary-encoded columns are not supported (write with use_dictionary=False)");
    std::size_t pos = static_cast<std::size_t>(c.data_page_offset);
    std::int64_t seen = 0;
    while (seen < c.num_values) {
      if (pos >= file.size()) return Fail(error, "parquet page offset is out of range");
      Thrift ph(file.data() + pos, file.size() - pos);
      int page_type = -1, uncompressed = 0, compressed = 0, num_values = 0, encoding = 0, def_encoding = 3;
      int pid = 0, pty = 0, plast = 0;
      while (ph.Field(&pid, &pty, &plast)) {
        if (pid == 1) page_type = static_cast<int>(ph.Zigzag());
        else if (pid == 2) uncompressed = static_cast<int>(ph.Zigzag());
        else if (pid == 3) compressed = static_cast<int>(ph.Zigzag());
        else if (pid == 5) {  // DataPageHeader
          int did = 0, dty = 0, dlast = 0;
          while (ph.Field(&did, &dty, &dlast)) {
            if (did == 1) num_values = static_cast<int>(ph.Zigzag());
            else if (did == 2) encoding = static_cast<int>(ph.Zigzag());
            else if (did == 3) def_encoding = static_cast<int>(ph.Zigzag());
            else ph.Skip(dty);
          }
        } else {
          ph.Skip(pty);
        }
      }
      if (!ph.ok()) return Fail(error, "parquet page header is malformed");
      const std::size_t body = static_cast<std::size_t>(ph.pos() - file.data());
      if (body + compressed > file.size()) return Fail(error, "parquet page is truncated");
      pos = body + compressed;
      if (page_type != 0) {
        if (page_type == 2) return Fail(error, "parquet dictionary pages are not supported");
        return Fail(error, "parquet DATA_PAGE_V2 and index pages are not supported");
      }
      if (encoding != 0) return Fail(error, "parquet data pages must use PLAIN encoding");
      std::vector<std::uint8_t> raw;
      const std::uint8_t* data = file.data() + body;
      std::size_t size = compressed;
      if (c.codec == 6) {
        raw.resize(uncompressed);
        if (!ZstdDecompress(data, compressed, &raw, error)) return false;
        data = raw.data();
        size = raw.size();
      }
      std::size_t off = 0;
      std::vector<std::uint8_t> defs;
      if (repetition == 1) {  // OPTIONAL: 4-byte length + RLE definition levels
        if (def_encoding != 3 || size < 4) return Fail(error, "parquet definition levels must be RLE");
        std::uint32_t len = 0;
        std::memcpy(&len, data, 4);
        if (4ull + len > size || !DecodeLevels(data + 4, len, num_values, &defs))
          return Fail(error, "parquet definition levels are malformed");
        off = 4 + len;
      }
      for (int i = 0; i < num_values; ++i) {
        if (repetition == 1 && defs[i] == 0) continue;  // null row
        if (off + 4 > size) return Fail(error, "parquet value stream is truncated");
        std::uint32_t len = 0;
        std::memcpy(&len, data + off, 4);
        off += 4;
        if (off + len > size) return Fail(error, "parquet value stream is truncated");
        out->emplace_back(reinterpret_cast<const char*>(data + off), len);
        off += len;
      }
      seen += num_values;
      if (num_values <= 0) break;
    }
  }
  return true;
}

}  // namespace ncb
