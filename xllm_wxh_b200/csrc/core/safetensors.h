// Memory-mapped safetensors reader.
//
// The reference parses the header through the Rust `safetensors` crate and wraps tensor
// bytes zero-copy (xllm/core/framework/state_dict/state_dict.cpp:122-262,
// state_dict/safetensors/src/lib.rs).  The format is: u64 little-endian header length,
// a JSON object {name: {dtype, shape, data_offsets:[begin,end]}, "__metadata__": {...}},
// then the raw tensor bytes.  The JSON subset used by the header is parsed here directly.
#pragma once
#include <fcntl.h>
#include <sys/mman.h>
#include <sys/stat.h>
#include <unistd.h>

#include <cstdint>
#include <cstring>
#include <map>
#include <stdexcept>
#include <string>
#include <vector>

namespace xl {

struct SafeTensorInfo {
  std::string name;
  std::string dtype;
  std::vector<int64_t> shape;
  uint64_t begin = 0, end = 0;  // offsets into the data section
};

class SafeTensorsFile {
 public:
  explicit SafeTensorsFile(const std::string& path) {
    fd_ = ::open(path.c_str(), O_RDONLY);
    if (fd_ < 0) throw std::runtime_error("cannot open " + path);
    struct stat st;
    if (fstat(fd_, &st) != 0 || st.st_size < 8) {
      ::close(fd_);
      throw std::runtime_error("bad safetensors file " + path);
    }
    size_ = static_cast<size_t>(st.st_size);
    base_ = static_cast<uint8_t*>(mmap(nullptr, size_, PROT_READ, MAP_PRIVATE, fd_, 0));
    if (base_ == MAP_FAILED) {
      ::close(fd_);
      throw std::runtime_error("mmap failed for " + path);
    }
    uint64_t hlen;
    std::memcpy(&hlen, base_, 8);
    if (hlen > size_ - 8) {
      cleanup();
      throw std::runtime_error("safetensors header length exceeds file size: " + path);
    }
    data_off_ = 8 + hlen;
    try {
      parse_header(reinterpret_cast<const char*>(base_ + 8), hlen);
    } catch (...) {
      cleanup();
      throw;
    }
    for (auto& kv : tensors_) {
      if (kv.second.end < kv.second.begin || data_off_ + kv.second.end > size_) {
        cleanup();
        throw std::runtime_error("tensor " + kv.first + " lies outside the file");
      }
    }
  }
  ~SafeTensorsFile() { cleanup(); }
  SafeTensorsFile(const SafeTensorsFile&) = delete;
  SafeTensorsFile& operator=(const SafeTensorsFile&) = delete;

  std::vector<std::string> keys() const {
    std::vector<std::string> k;
    for (auto& kv : tensors_) k.push_back(kv.first);
    return k;
  }
  bool has(const std::string& name) const { return tensors_.count(name) > 0; }
  const SafeTensorInfo& info(const std::string& name) const {
    auto it = tensors_.find(name);
    if (it == tensors_.end()) throw std::out_of_range("no tensor named " + name);
    return it->second;
  }
  const std::map<std::string, std::string>& metadata() const { return metadata_; }
  uint8_t* data() const { return base_ + data_off_; }
  size_t data_size() const { return size_ - data_off_; }

 private:
  void cleanup() {
    if (base_ && base_ != MAP_FAILED) munmap(base_, size_);
    base_ = nullptr;
    if (fd_ >= 0) ::close(fd_);
    fd_ = -1;
  }

  // --- minimal JSON reader for the header subset
  struct Cur {
    const char* p;
    const char* e;
  };
  static void ws(Cur& c) {
    while (c.p < c.e && (*c.p == ' ' || *c.p == '\n' || *c.p == '\t' || *c.p == '\r')) ++c.p;
  }
  static void expect(Cur& c, char ch) {
    ws(c);
    if (c.p >= c.e || *c.p != ch) throw std::runtime_error(std::string("safetensors header: expected '") + ch + "'");
    ++c.p;
  }
  static std::string str(Cur& c) {
    expect(c, '"');
    std::string out;
    while (c.p < c.e && *c.p != '"') {
      if (*c.p == '\\' && c.p + 1 < c.e) {
        ++c.p;
        switch (*c.p) {
          case 'n': out += '\n'; break;
          case 't': out += '\t'; break;
          case 'r': out += '\r'; break;
          case 'b': out += '\b'; break;
          case 'f': out += '\f'; break;
          case 'u': {
            if (c.p + 4 >= c.e) throw std::runtime_error("bad \\u escape");
            unsigned v = std::stoul(std::string(c.p + 1, c.p + 5), nullptr, 16);
            c.p += 4;
            if (v < 0x80) out += char(v);
            else if (v < 0x800) { out += char(0xC0 | (v >> 6)); out += char(0x80 | (v & 0x3F)); }
            else { out += char(0xE0 | (v >> 12)); out += char(0x80 | ((v >> 6) & 0x3F)); out += char(0x80 | (v & 0x3F)); }
            break;
          }
          default: out += *c.p;
        }
        ++c.p;
      } else {
        out += *c.p++;
      }
    }
    expect(c, '"');
    return out;
  }
  static int64_t num(Cur& c) {
    ws(c);
    const char* s = c.p;
    while (c.p < c.e && (*c.p == '-' || (*c.p >= '0' && *c.p <= '9'))) ++c.p;
    if (s == c.p) throw std::runtime_error("safetensors header: expected number");
    return std::stoll(std::string(s, c.p));
  }
  static void skip_value(Cur& c) {
    ws(c);
    if (c.p >= c.e) return;
    if (*c.p == '"') { str(c); return; }
    if (*c.p == '{' || *c.p == '[') {
      char open = *c.p, close = (open == '{') ? '}' : ']';
      ++c.p;
      ws(c);
      if (c.p < c.e && *c.p == close) { ++c.p; return; }
      while (true) {
        if (open == '{') { str(c); expect(c, ':'); }
        skip_value(c);
        ws(c);
        if (c.p < c.e && *c.p == ',') { ++c.p; continue; }
        expect(c, close);
        return;
      }
    }
    while (c.p < c.e && *c.p != ',' && *c.p != '}' && *c.p != ']') ++c.p;
  }

  void parse_header(const char* s, size_t n) {
    Cur c{s, s + n};
    expect(c, '{');
    ws(c);
    if (c.p < c.e && *c.p == '}') return;
    while (true) {
      std::string name = str(c);
      expect(c, ':');
      if (name == "__metadata__") {
        expect(c, '{');
        ws(c);
        if (c.p < c.e && *c.p == '}') {
          ++c.p;
        } else {
          while (true) {
            std::string k = str(c);
            expect(c, ':');
            ws(c);
            if (c.p < c.e && *c.p == '"') metadata_[k] = str(c); else skip_value(c);
            ws(c);
            if (c.p < c.e && *c.p == ',') { ++c.p; continue; }
            expect(c, '}');
            break;
          }
        }
      } else {
        SafeTensorInfo ti;
        ti.name = name;
        expect(c, '{');
        while (true) {
          std::string k = str(c);
          expect(c, ':');
          if (k == "dtype") {
            ti.dtype = str(c);
          } else if (k == "shape") {
            expect(c, '[');
            ws(c);
            if (c.p < c.e && *c.p == ']') {
              ++c.p;
            } else {
              while (true) {
                ti.shape.push_back(num(c));
                ws(c);
                if (c.p < c.e && *c.p == ',') { ++c.p; continue; }
                expect(c, ']');
                break;
              }
            }
          } else if (k == "data_offsets") {
            expect(c, '[');
            ti.begin = static_cast<uint64_t>(num(c));
            expect(c, ',');
            ti.end = static_cast<uint64_t>(num(c));
            expect(c, ']');
          } else {
            skip_value(c);
          }
          ws(c);
          if (c.p < c.e && *c.p == ',') { ++c.p; continue; }
          expect(c, '}');
          break;
        }
        tensors_[name] = std::move(ti);
      }
      ws(c);
      if (c.p < c.e && *c.p == ',') { ++c.p; continue; }
      expect(c, '}');
      break;
    }
  }

  int fd_ = -1;
  uint8_t* base_ = nullptr;
  size_t size_ = 0, data_off_ = 0;
  std::map<std::string, SafeTensorInfo> tensors_;
  std::map<std::string, std::string> metadata_;
};

}  // namespace xl
