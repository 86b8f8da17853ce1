// Weights checkpoint I/O in the reference's format (crates/pm-train/src/checkpoint.rs:25-97): a safetensors file
// whose tensors are the model parameters by position, named "p_0000", "p_0001", ... in `append_params` order, all
// F32.  Load insists on the same count, dtype and shapes, like the reference.
//
// safetensors layout: 8 bytes little-endian header length N, N bytes of JSON
//   {"p_0000":{"dtype":"F32","shape":[..],"data_offsets":[begin,end]}, ... , optional "__metadata__":{..}}
// followed by one byte buffer; offsets are relative to its start.  The writer emits the tensors in name order,
// back to back, and pads the header with spaces to a multiple of 8 bytes, which is what the reference's serializer
// produces for tensors of one dtype.  The reader accepts any order and any metadata.
#include <cerrno>
#include <cstdio>
#include <cstring>
#include <map>
#include <string>
#include <vector>
#include "common.cuh"

namespace pmb {
namespace {

struct Entry { std::string dtype; std::vector<int64_t> shape; uint64_t begin = 0, end = 0; };

// Minimal JSON reader for the header: objects, arrays, strings (with the standard escapes), integers; anything else
// inside "__metadata__" is skipped structurally.
struct Json {
  const char* p; const char* e; bool ok = true;
  void ws() { while (p < e && (*p == ' ' || *p == '\n' || *p == '\t' || *p == '\r')) ++p; }
  bool eat(char c) { ws(); if (p < e && *p == c) { ++p; return true; } return false; }
  bool str(std::string* out) {
    ws();
    if (p >= e || *p != '"') return ok = false;
    ++p;
    std::string s;
    while (p < e && *p != '"') {
      if (*p == '\\') {
        if (++p >= e) return ok = false;
        switch (*p) {
          case 'n': s += '\n'; break; case 't': s += '\t'; break; case 'r': s += '\r'; break;
          case 'b': s += '\b'; break; case 'f': s += '\f'; break;
          case 'u': if (e - p < 5) return ok = false; s += '?'; p += 4; break;   // names here are ASCII
          default: s += *p;
        }
        ++p;
      } else {
        s += *p++;
      }
    }
    if (p >= e) return ok = false;
    ++p;
    if (out) *out = s;
    return true;
  }
  bool num(int64_t* out) {
    ws();
    const char* b = p;
    if (p < e && *p == '-') ++p;
    int64_t v = 0; bool any = false;
    while (p < e && *p >= '0' && *p <= '9') { v = v * 10 + (*p - '0'); ++p; any = true; }
    if (!any) return ok = false;
    if (out) *out = (*b == '-') ? -v : v;
    return true;
  }
  bool skip() {   // any value
    ws();
    if (p >= e) return ok = false;
    if (*p == '"') return str(nullptr);
    if (*p == '{') {
      ++p;
      if (eat('}')) return true;
      do { if (!str(nullptr) || !eat(':') || !skip()) return ok = false; } while (eat(','));
      return eat('}') ? true : (ok = false);
    }
    if (*p == '[') {
      ++p;
      if (eat(']')) return true;
      do { if (!skip()) return ok = false; } while (eat(','));
      return eat(']') ? true : (ok = false);
    }
    while (p < e && *p != ',' && *p != '}' && *p != ']') ++p;   // number / true / false / null
    return true;
  }
};

bool parse_header(const char* b, const char* e, std::map<std::string, Entry>* out) {
  Json j{b, e};
  if (!j.eat('{')) return false;
  if (j.eat('}')) return true;
  do {
    std::string name;
    if (!j.str(&name) || !j.eat(':')) return false;
    if (name == "__metadata__") { if (!j.skip()) return false; continue; }
    Entry en;
    if (!j.eat('{')) return false;
    do {
      std::string key;
      if (!j.str(&key) || !j.eat(':')) return false;
      if (key == "dtype") { if (!j.str(&en.dtype)) return false; }
      else if (key == "shape" || key == "data_offsets") {
        std::vector<int64_t> v;
        if (!j.eat('[')) return false;
        if (!j.eat(']')) {
          do { int64_t x; if (!j.num(&x)) return false; v.push_back(x); } while (j.eat(','));
          if (!j.eat(']')) return false;
        }
        if (key == "shape") en.shape = v;
        else { if (v.size() != 2 || v[0] < 0 || v[1] < v[0]) return false; en.begin = (uint64_t)v[0]; en.end = (uint64_t)v[1]; }
      } else if (!j.skip()) return false;
    } while (j.eat(','));
    if (!j.eat('}')) return false;
    (*out)[name] = en;
  } while (j.eat(','));
  return j.eat('}') && j.ok;
}

std::string tensor_name(int i) { char b[32]; snprintf(b, sizeof b, "p_%04d", i); return b; }

}  // namespace

pmb_status safetensors_save_f32(const char* path, int n, const int64_t* shapes, const int32_t* ranks, const float* const* data) {
  if (!path || n < 0 || (n > 0 && (!shapes || !ranks || !data))) return fail(PMB_ERR_ARG, "safetensors_save: bad argument");
  std::string hdr = "{";
  uint64_t off = 0;
  std::vector<uint64_t> bytes(n);
  const int64_t* sp = shapes;
  for (int i = 0; i < n; ++i) {
    uint64_t el = 1;
    std::string sh = "[";
    for (int r = 0; r < ranks[i]; ++r) {
      if (sp[r] < 0) return fail(PMB_ERR_SHAPE, "safetensors_save: negative extent");
      el *= (uint64_t)sp[r];
      sh += std::to_string(sp[r]);
      if (r + 1 < ranks[i]) sh += ",";
    }
    sh += "]";
    sp += ranks[i];
    bytes[i] = el * 4;
    if (i) hdr += ",";
    hdr += "\"" + tensor_name(i) + "\":{\"dtype\":\"F32\",\"shape\":" + sh + ",\"data_offsets\":[" + std::to_string(off) + "," +
           std::to_string(off + bytes[i]) + "]}";
    off += bytes[i];
  }
  hdr += "}";
  while (hdr.size() % 8) hdr += ' ';
  FILE* f = fopen(path, "wb");
  if (!f) return fail(PMB_ERR_ARG, "safetensors_save: cannot open %s: %s", path, strerror(errno));
  const uint64_t hlen = hdr.size();
  unsigned char lenb[8];
  for (int i = 0; i < 8; ++i) lenb[i] = (unsigned char)((hlen >> (8 * i)) & 0xff);
  bool ok = fwrite(lenb, 1, 8, f) == 8 && fwrite(hdr.data(), 1, hdr.size(), f) == hdr.size();
  for (int i = 0; i < n && ok; ++i) ok = bytes[i] == 0 || fwrite(data[i], 1, bytes[i], f) == bytes[i];
  ok = (fclose(f) == 0) && ok;
  if (!ok) return fail(PMB_ERR_ARG, "safetensors_save: short write to %s", path);
  return PMB_OK;
}

pmb_status safetensors_load_f32(const char* path, int n, const int64_t* shapes, const int32_t* ranks, float* const* data) {
  if (!path || n < 0 || (n > 0 && (!shapes || !ranks || !data))) return fail(PMB_ERR_ARG, "safetensors_load: bad argument");
  FILE* f = fopen(path, "rb");
  if (!f) return fail(PMB_ERR_ARG, "safetensors_load: cannot open %s: %s", path, strerror(errno));
  unsigned char lenb[8];
  if (fread(lenb, 1, 8, f) != 8) { fclose(f); return fail(PMB_ERR_ARG, "safetensors_load: %s is shorter than its length field", path); }
  uint64_t hlen = 0;
  for (int i = 0; i < 8; ++i) hlen |= (uint64_t)lenb[i] << (8 * i);
  if (hlen > (100u << 20)) { fclose(f); return fail(PMB_ERR_ARG, "safetensors_load: header of %llu bytes is not plausible", (unsigned long long)hlen); }
  std::string hdr(hlen, '\0');
  if (fread(&hdr[0], 1, hlen, f) != hlen) { fclose(f); return fail(PMB_ERR_ARG, "safetensors_load: truncated header in %s", path); }
  std::map<std::string, Entry> ent;
  if (!parse_header(hdr.data(), hdr.data() + hdr.size(), &ent)) { fclose(f); return fail(PMB_ERR_ARG, "safetensors_load: malformed header in %s", path); }
  if ((int)ent.size() != n) {
    fclose(f);
    return fail(PMB_ERR_SHAPE, "checkpoint has %zu tensors, model has %d params", ent.size(), n);
  }
  const long data0 = 8 + (long)hlen;
  const int64_t* sp = shapes;
  pmb_status st = PMB_OK;
  for (int i = 0; i < n && st == PMB_OK; ++i) {
    const std::string name = tensor_name(i);
    auto it = ent.find(name);
    std::vector<int64_t> want(sp, sp + ranks[i]);
    sp += ranks[i];
    if (it == ent.end()) { st = fail(PMB_ERR_SHAPE, "tensor %s: not in the checkpoint", name.c_str()); break; }
    const Entry& en = it->second;
    if (en.dtype != "F32") { st = fail(PMB_ERR_UNSUPPORTED, "param %s: expected F32, got %s", name.c_str(), en.dtype.c_str()); break; }
    if (en.shape != want) { st = fail(PMB_ERR_SHAPE, "param %s: shape mismatch between file and model", name.c_str()); break; }
    uint64_t el = 1;
    for (int64_t x : want) el *= (uint64_t)x;
    if (en.end - en.begin != el * 4) { st = fail(PMB_ERR_SHAPE, "param %s: data_offsets do not match its shape", name.c_str()); break; }
    if (el == 0) continue;
    if (fseek(f, data0 + (long)en.begin, SEEK_SET) != 0 || fread(data[i], 1, el * 4, f) != el * 4)
      st = fail(PMB_ERR_ARG, "param %s: file ends inside its data", name.c_str());
  }
  fclose(f);
  return st;
}

}  // namespace pmb

extern "C" pmb_status pmb_safetensors_save_f32(const char* path, int32_t n_tensors, const int64_t* shapes_flat, const int32_t* ranks,
                                               const float* const* h_data) {
  return pmb::safetensors_save_f32(path, n_tensors, shapes_flat, ranks, h_data);
}

extern "C" pmb_status pmb_safetensors_load_f32(const char* path, int32_t n_tensors, const int64_t* shapes_flat, const int32_t* ranks,
                                               float* const* h_data) {
  return pmb::safetensors_load_f32(path, n_tensors, shapes_flat, ranks, h_data);
}
