// `.fst` reader for the MLA tensors: see fst_file.h for the layout and the reference lines.
#include "fst_file.h"

#include <cmath>
#include <cstdio>
#include <cstring>
#include <stdexcept>

namespace fstfile {

namespace {

struct File {
  FILE* f = nullptr;
  std::string path;
  explicit File(const std::string& p) : f(std::fopen(p.c_str(), "rb")), path(p) {
    if (!f) throw std::runtime_error(p + ": cannot open");
  }
  ~File() {
    if (f) std::fclose(f);
  }
  uint64_t size() {
    std::fseek(f, 0, SEEK_END);
    const long n = std::ftell(f);
    return n < 0 ? 0 : (uint64_t)n;
  }
  std::vector<unsigned char> read(uint64_t off, uint64_t n, const char* what) {
    std::vector<unsigned char> buf(n);
    if (std::fseek(f, (long)off, SEEK_SET) != 0 || (n && std::fread(buf.data(), 1, n, f) != n))
      throw std::runtime_error(path + ": " + what + " is cut short");
    return buf;
  }
};

template <typename T>
T get(const unsigned char* p) {
  T v;
  std::memcpy(&v, p, sizeof(T));
  return v;
}

float half_to_float(uint16_t h) {
  const uint32_t sign = (uint32_t)(h & 0x8000u) << 16, exp = (h >> 10) & 0x1Fu, man = h & 0x3FFu;
  uint32_t bits;
  if (exp == 0) {
    if (man == 0) {
      bits = sign;
    } else {  // subnormal half: value = man * 2^-24
      float v = std::ldexp((float)man, -24);
      std::memcpy(&bits, &v, 4);
      bits |= sign;
    }
  } else if (exp == 31) {
    bits = sign | 0x7F800000u | (man << 13);
  } else {
    bits = sign | ((exp + 112u) << 23) | (man << 13);
  }
  float out;
  std::memcpy(&out, &bits, 4);
  return out;
}

uint16_t trunc_bf16(float v) {  // the reference's f2bf truncates (src/fst_engine.cpp:27)
  uint32_t b;
  std::memcpy(&b, &v, 4);
  return (uint16_t)(b >> 16);
}

float widen_bf16(uint16_t b) {
  const uint32_t u = (uint32_t)b << 16;
  float v;
  std::memcpy(&v, &u, 4);
  return v;
}

// the values of an entry as fp32 (Q8_0 expanded), or as raw bf16 bits when the payload is BF16
void load(const std::string& path, const Entry& e, std::vector<float>* f32, std::vector<uint16_t>* bits) {
  File file(path);
  const std::vector<unsigned char> raw = file.read(e.offset, e.size, "a tensor payload");
  const uint64_t n = e.n_elements();
  if (e.qtype == QTYPE_BF16) {
    if (e.size < 2 * n) throw std::runtime_error(path + ": BF16 payload smaller than its shape");
    bits->resize(n);
    std::memcpy(bits->data(), raw.data(), 2 * n);
  } else if (e.qtype == QTYPE_F32) {
    if (e.size < 4 * n) throw std::runtime_error(path + ": F32 payload smaller than its shape");
    f32->resize(n);
    std::memcpy(f32->data(), raw.data(), 4 * n);
  } else if (e.qtype == QTYPE_Q8_0) {
    const uint64_t nb = (n + 31) / 32;
    if (e.size < nb * 34) throw std::runtime_error(path + ": Q8_0 payload smaller than its shape");
    const unsigned char* q = raw.data() + nb * 2;
    f32->resize(n);
    for (uint64_t b = 0; b < nb; ++b) {
      float s = half_to_float(get<uint16_t>(raw.data() + 2 * b));
      if (std::fabs(s) < 1e-12f) s = 1.0f;  // src/fst_engine.cpp:1595
      for (uint64_t j = 0; j < 32 && b * 32 + j < n; ++j) (*f32)[b * 32 + j] = (float)(int8_t)q[b * 32 + j] * s;
    }
  } else {
    throw std::runtime_error(path + ": unknown qtype " + std::to_string(e.qtype));
  }
}

}  // namespace

uint64_t Entry::n_elements() const {
  uint64_t n = 1;
  for (int i = 0; i < ndim && i < 3; ++i) n *= shape[i];
  return n;
}

Header read_header(const std::string& path) {
  File file(path);
  if (file.size() < 128) throw std::runtime_error(path + ": shorter than a 128-byte header");
  const std::vector<unsigned char> h = file.read(0, 128, "the header");
  if (std::memcmp(h.data(), "FST\0", 4) != 0) throw std::runtime_error(path + ": bad magic");
  Header o;
  // "<4sIIIIIIIIIIIQffQQ...": eleven u32 after the version, then u64 vocab, two f32, u64 offset, u64 count
  o.version = get<uint32_t>(&h[4]);
  o.hidden_dim = get<uint32_t>(&h[8]);
  o.n_layers = get<uint32_t>(&h[12]);
  o.n_experts = get<uint32_t>(&h[16]);
  o.top_k = get<uint32_t>(&h[20]);
  o.n_q_heads = get<uint32_t>(&h[24]);
  o.n_kv_heads = get<uint32_t>(&h[28]);
  o.head_dim = get<uint32_t>(&h[32]);
  o.vocab_size = get<uint64_t>(&h[48]);
  o.rms_eps = get<float>(&h[56]);
  o.rope_freq_base = get<float>(&h[60]);
  if (!(o.rope_freq_base > 0.0f)) o.rope_freq_base = 10000.0f;  // src/fst_engine.cpp:1505
  o.dir_offset = get<uint64_t>(&h[64]);
  o.dir_count = get<uint64_t>(&h[72]);
  return o;
}

std::vector<Entry> read_directory(const std::string& path, Header* header_out) {
  const Header h = read_header(path);
  if (header_out) *header_out = h;
  File file(path);
  const uint64_t fsize = file.size();
  if (h.dir_count > (1u << 24) || h.dir_offset + h.dir_count * 64 > fsize)
    throw std::runtime_error(path + ": the directory is cut short");
  const std::vector<unsigned char> raw = file.read(h.dir_offset, h.dir_count * 64, "the directory");
  std::vector<Entry> out(h.dir_count);
  for (uint64_t i = 0; i < h.dir_count; ++i) {
    const unsigned char* p = raw.data() + i * 64;  // "<IHHHHIQQQQQQ"
    Entry& e = out[i];
    e.tid = get<uint32_t>(p);
    e.layer = get<uint16_t>(p + 4);
    e.sub = get<uint16_t>(p + 6);
    e.qtype = get<uint16_t>(p + 8);
    e.ndim = get<uint16_t>(p + 10);
    for (int k = 0; k < 3; ++k) e.shape[k] = get<uint64_t>(p + 16 + 8 * k);
    e.offset = get<uint64_t>(p + 40);
    e.size = get<uint64_t>(p + 48);
    if (e.ndim > 3 || e.offset + e.size > fsize)
      throw std::runtime_error(path + ": entry " + std::to_string(i) + " is out of bounds");
  }
  return out;
}

const Entry* find(const std::vector<Entry>& dir, uint32_t tid, int layer, int sub) {
  for (const Entry& e : dir)
    if (e.tid == tid && e.sub == sub && (e.layer == layer || e.layer == GLOBAL_LAYER)) return &e;
  return nullptr;
}

const Entry* find_shape(const std::vector<Entry>& dir, uint32_t tid, int layer, uint64_t s0, uint64_t s1) {
  for (const Entry& e : dir)
    if (e.tid == tid && (e.layer == layer || e.layer == GLOBAL_LAYER) && e.ndim >= 1 && e.shape[0] == s0 &&
        (e.ndim >= 2 ? e.shape[1] : 1) == s1)
      return &e;
  return nullptr;
}

std::vector<uint16_t> load_bf16(const std::string& path, const Entry& e) {
  std::vector<float> f;
  std::vector<uint16_t> b;
  load(path, e, &f, &b);
  if (e.qtype != QTYPE_BF16) {
    b.resize(f.size());
    for (size_t i = 0; i < f.size(); ++i) b[i] = trunc_bf16(f[i]);
  }
  return b;
}

std::vector<float> load_f32(const std::string& path, const Entry& e) {
  std::vector<float> f;
  std::vector<uint16_t> b;
  load(path, e, &f, &b);
  if (e.qtype == QTYPE_BF16) {
    f.resize(b.size());
    for (size_t i = 0; i < b.size(); ++i) f[i] = widen_bf16(b[i]);
  }
  return f;
}

}  // namespace fstfile
