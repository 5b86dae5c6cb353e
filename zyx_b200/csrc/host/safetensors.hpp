// safetensors files, read and written the way the reference does (Module::save, zyx/src/module.rs:36-63;
// Tensor::load_safetensors, module.rs:436-529), used by the C entry points zyxb_st_* and by the plans' checkpoints.
#pragma once
#include <stdint.h>
#include <stdio.h>

#include <string>
#include <vector>

#include "../../../include/zyxb.h"

namespace zyxb_host {
namespace st {

struct TensorRef {
  std::string name;
  int32_t dtype = ZYXB_F32;
  std::vector<uint64_t> shape;
  const void* data = nullptr;
};
struct Entry {
  std::string name;
  int32_t dtype = ZYXB_F32;
  std::vector<uint64_t> shape;
  uint64_t begin = 0, end = 0;      // data_offsets, relative to the end of the header
};
struct File {
  FILE* f = nullptr;
  uint64_t data_start = 0, data_bytes = 0;
  std::vector<Entry> entries;       // in header order
};

// DType::safetensors / from_safetensors (zyx/src/dtype.rs:227-262)
inline const char* dtype_name(int32_t d) {
  switch (d) {
    case ZYXB_BF16: return "BF16"; case ZYXB_F16: return "F16"; case ZYXB_F32: return "F32"; case ZYXB_F64: return "F64";
    case ZYXB_U8: return "U8"; case ZYXB_U16: return "U16"; case ZYXB_U32: return "U32"; case ZYXB_U64: return "U64";
    case ZYXB_I8: return "I8"; case ZYXB_I16: return "I16"; case ZYXB_I32: return "I32"; case ZYXB_I64: return "I64";
    case ZYXB_BOOL: return "BOOL"; default: return nullptr;
  }
}
inline int32_t dtype_from_name(const std::string& s) {
  for (int32_t d = ZYXB_BF16; d <= ZYXB_BOOL; ++d)
    if (s == dtype_name(d)) return d;
  return -1;
}
inline uint64_t dtype_bytes(int32_t d) {
  switch (d) {
    case ZYXB_BF16: case ZYXB_F16: case ZYXB_U16: case ZYXB_I16: return 2;
    case ZYXB_F32: case ZYXB_U32: case ZYXB_I32: return 4;
    case ZYXB_F64: case ZYXB_U64: case ZYXB_I64: return 8;
    default: return 1;
  }
}
// Saturating: a crafted header (shape [2^63, 2]) must not wrap around into a small element count that passes the
// shape / data_offsets check.
inline uint64_t numel(const std::vector<uint64_t>& shape) {
  uint64_t n = 1;
  for (uint64_t d : shape) if (__builtin_mul_overflow(n, d, &n)) return UINT64_MAX / 16;
  return n;
}

inline void json_escape(const std::string& in, std::string& out) {
  for (unsigned char c : in) {
    if (c == '"' || c == '\\') { out.push_back('\\'); out.push_back((char)c); }
    else if (c < 0x20) { char b[8]; snprintf(b, sizeof b, "\\u%04x", c); out += b; }
    else out.push_back((char)c);
  }
}

inline bool write(const std::string& path, const std::vector<TensorRef>& tensors, std::string& err) {
  std::string header = "{";
  uint64_t begin = 0;
  for (const TensorRef& t : tensors) {
    const char* dn = dtype_name(t.dtype);
    if (!dn) { err = "safetensors: tensor '" + t.name + "' has an unknown dtype"; return false; }
    const uint64_t bytes = numel(t.shape) * dtype_bytes(t.dtype);
    header += "\"";
    json_escape(t.name, header);
    header += "\":{\"dtype\":\"";
    header += dn;
    header += "\",\"shape\":[";
    for (size_t i = 0; i < t.shape.size(); ++i) { if (i) header += ","; header += std::to_string(t.shape[i]); }
    header += "],\"data_offsets\":[" + std::to_string(begin) + "," + std::to_string(begin + bytes) + "]},";
    begin += bytes;
  }
  if (header.size() > 1) header.pop_back();
  header += "}";
  FILE* f = fopen(path.c_str(), "wb");
  if (!f) { err = "safetensors: cannot create " + path; return false; }
  const uint64_t n = header.size();
  unsigned char len[8];
  for (int i = 0; i < 8; ++i) len[i] = (unsigned char)(n >> (8 * i));
  bool ok = fwrite(len, 1, 8, f) == 8 && fwrite(header.data(), 1, header.size(), f) == header.size();
  for (const TensorRef& t : tensors) {
    const uint64_t bytes = numel(t.shape) * dtype_bytes(t.dtype);
    if (ok && bytes) ok = fwrite(t.data, 1, bytes, f) == bytes;
  }
  ok = (fclose(f) == 0) && ok;
  if (!ok) err = "safetensors: write to " + path + " failed";
  return ok;
}

// ---- a small JSON reader: just enough for a safetensors header, tolerant of anything valid it does not need ----
struct Json {
  const std::string& s;
  size_t i = 0;
  std::string err;
  explicit Json(const std::string& text) : s(text) {}
  void ws() { while (i < s.size() && (s[i] == ' ' || s[i] == '\n' || s[i] == '\t' || s[i] == '\r')) ++i; }
  bool fail(const char* what) { if (err.empty()) err = std::string("safetensors header: ") + what + " at byte " + std::to_string(i); return false; }
  bool expect(char c) { ws(); if (i < s.size() && s[i] == c) { ++i; return true; } return fail("unexpected character"); }
  bool peek(char c) { ws(); return i < s.size() && s[i] == c; }
  bool string(std::string& out) {
    out.clear();
    if (!expect('"')) return false;
    while (i < s.size() && s[i] != '"') {
      if (s[i] == '\\') {
        if (++i >= s.size()) return fail("truncated escape");
        switch (s[i]) {
          case 'n': out.push_back('\n'); break; case 't': out.push_back('\t'); break; case 'r': out.push_back('\r'); break;
          case 'b': out.push_back('\b'); break; case 'f': out.push_back('\f'); break;
          case 'u': {
            if (i + 4 >= s.size()) return fail("truncated \\u escape");
            const unsigned v = (unsigned)strtoul(s.substr(i + 1, 4).c_str(), nullptr, 16);
            if (v < 0x80) out.push_back((char)v);
            else if (v < 0x800) { out.push_back((char)(0xc0 | (v >> 6))); out.push_back((char)(0x80 | (v & 0x3f))); }
            else { out.push_back((char)(0xe0 | (v >> 12))); out.push_back((char)(0x80 | ((v >> 6) & 0x3f))); out.push_back((char)(0x80 | (v & 0x3f))); }
            i += 4;
            break;
          }
          default: out.push_back(s[i]);
        }
        ++i;
      } else out.push_back(s[i++]);
    }
    return expect('"');
  }
  bool uint(uint64_t& out) {
    ws();
    if (i >= s.size() || s[i] < '0' || s[i] > '9') return fail("expected a non-negative integer");
    out = 0;
    while (i < s.size() && s[i] >= '0' && s[i] <= '9') {
      if (out > (UINT64_MAX - 9) / 10) return fail("integer too large");
      out = out * 10 + (uint64_t)(s[i++] - '0');
    }
    return true;
  }
  bool uint_array(std::vector<uint64_t>& out) {
    out.clear();
    if (!expect('[')) return false;
    if (peek(']')) { ++i; return true; }
    for (;;) {
      uint64_t v;
      if (!uint(v)) return false;
      out.push_back(v);
      if (peek(',')) { ++i; continue; }
      return expect(']');
    }
  }
  bool skip_value() {   // any JSON value
    ws();
    if (i >= s.size()) return fail("truncated value");
    if (s[i] == '"') { std::string t; return string(t); }
    if (s[i] == '{' || s[i] == '[') {
      const char close = s[i] == '{' ? '}' : ']';
      ++i;
      if (peek(close)) { ++i; return true; }
      for (;;) {
        if (close == '}') { std::string k; if (!string(k) || !expect(':')) return false; }
        if (!skip_value()) return false;
        if (peek(',')) { ++i; continue; }
        return expect(close);
      }
    }
    while (i < s.size() && s[i] != ',' && s[i] != '}' && s[i] != ']') ++i;   // number, true, false, null
    return true;
  }
};

inline bool parse_header(const std::string& header, uint64_t data_bytes, std::vector<Entry>& entries, std::string& err) {
  Json j(header);
  entries.clear();
  if (!j.expect('{')) { err = j.err; return false; }
  if (j.peek('}')) return true;
  for (;;) {
    Entry e;
    bool have_dtype = false, have_shape = false, have_off = false;
    if (!j.string(e.name) || !j.expect(':')) { err = j.err; return false; }
    if (e.name == "__metadata__") {
      if (!j.skip_value()) { err = j.err; return false; }
    } else {
      if (!j.expect('{')) { err = j.err; return false; }
      for (;;) {
        std::string key;
        if (!j.string(key) || !j.expect(':')) { err = j.err; return false; }
        if (key == "dtype") {
          std::string d;
          if (!j.string(d)) { err = j.err; return false; }
          e.dtype = dtype_from_name(d);
          if (e.dtype < 0) { err = "safetensors: tensor '" + e.name + "' has unsupported dtype " + d; return false; }
          have_dtype = true;
        } else if (key == "shape") {
          if (!j.uint_array(e.shape)) { err = j.err; return false; }
          have_shape = true;
        } else if (key == "data_offsets") {
          std::vector<uint64_t> o;
          if (!j.uint_array(o)) { err = j.err; return false; }
          if (o.size() != 2) { err = "safetensors: data_offsets of '" + e.name + "' must hold two numbers"; return false; }
          e.begin = o[0]; e.end = o[1];
          have_off = true;
        } else if (!j.skip_value()) { err = j.err; return false; }
        if (j.peek(',')) { ++j.i; continue; }
        if (!j.expect('}')) { err = j.err; return false; }
        break;
      }
      if (!have_dtype || !have_shape || !have_off) { err = "safetensors: tensor '" + e.name + "' lacks dtype, shape or data_offsets"; return false; }
      // the reference's check (module.rs:506-509), plus the bounds of the file
      if (e.end < e.begin || e.end - e.begin != numel(e.shape) * dtype_bytes(e.dtype)) {
        err = "safetensors: shape and offsets of '" + e.name + "' disagree"; return false;
      }
      if (e.end > data_bytes) { err = "safetensors: '" + e.name + "' extends past the end of the file"; return false; }
      entries.push_back(std::move(e));
    }
    if (j.peek(',')) { ++j.i; continue; }
    if (!j.expect('}')) { err = j.err; return false; }
    return true;
  }
}

inline void close(File& f) {
  if (f.f) fclose(f.f);
  f.f = nullptr;
}
inline bool open(const std::string& path, File& out, std::string& err) {
  FILE* f = fopen(path.c_str(), "rb");
  if (!f) { err = "safetensors: cannot open " + path; return false; }
  unsigned char len[8];
  if (fread(len, 1, 8, f) != 8) { fclose(f); err = "safetensors: " + path + " is shorter than its header length field"; return false; }
  uint64_t n = 0;
  for (int i = 0; i < 8; ++i) n |= (uint64_t)len[i] << (8 * i);
  fseek(f, 0, SEEK_END);
  const uint64_t total = (uint64_t)ftell(f);
  if (n > total - 8 || n > (1ull << 30)) { fclose(f); err = "safetensors: header length " + std::to_string(n) + " exceeds the file"; return false; }
  std::string header(n, '\0');
  fseek(f, 8, SEEK_SET);
  if (n && fread(&header[0], 1, n, f) != n) { fclose(f); err = "safetensors: cannot read the header of " + path; return false; }
  out.f = f; out.data_start = 8 + n; out.data_bytes = total - out.data_start;
  if (!parse_header(header, out.data_bytes, out.entries, err)) { close(out); return false; }
  return true;
}
inline int find(const File& f, const std::string& name) {
  for (size_t i = 0; i < f.entries.size(); ++i)
    if (f.entries[i].name == name) return (int)i;
  return -1;
}
inline bool read(File& f, int i, void* dst, uint64_t dst_bytes, std::string& err) {
  if (!f.f || i < 0 || (size_t)i >= f.entries.size()) { err = "safetensors: no such tensor"; return false; }
  const Entry& e = f.entries[i];
  const uint64_t bytes = e.end - e.begin;
  if (dst_bytes < bytes) { err = "safetensors: destination for '" + e.name + "' is too small"; return false; }
  if (fseek(f.f, (long)(f.data_start + e.begin), SEEK_SET) != 0 || (bytes && fread(dst, 1, bytes, f.f) != bytes)) {
    err = "safetensors: cannot read '" + e.name + "'"; return false;
  }
  return true;
}

}  // namespace st
}  // namespace zyxb_host
