#include "host/mllm_file.h"

#include <fcntl.h>
#include <sys/mman.h>
#include <sys/stat.h>
#include <unistd.h>

#include <algorithm>
#include <cstring>
#include <fstream>
#include <stdexcept>
#include <thread>

namespace mb200host {
namespace {

constexpr int32_t kMagicV1 = 20012;
constexpr int32_t kMagicV2 = 0x519A;
constexpr uint64_t kV2Header = 532;
constexpr uint64_t kV2Desc = 352;

template <typename T>
T rd(const uint8_t* p) {
  T v;
  std::memcpy(&v, p, sizeof(T));
  return v;
}

float half_to_float(uint16_t h) {
  const uint32_t sign = (h & 0x8000u) << 16;
  uint32_t exp = (h >> 10) & 0x1F;
  uint32_t man = h & 0x3FF;
  uint32_t bits;
  if (exp == 0) {
    if (man == 0) {
      bits = sign;
    } else {  // subnormal
      exp = 127 - 15 + 1;
      while ((man & 0x400) == 0) {
        man <<= 1;
        --exp;
      }
      man &= 0x3FF;
      bits = sign | (exp << 23) | (man << 13);
    }
  } else if (exp == 31) {
    bits = sign | 0x7F800000u | (man << 13);
  } else {
    bits = sign | ((exp + 127 - 15) << 23) | (man << 13);
  }
  float f;
  std::memcpy(&f, &bits, 4);
  return f;
}

// ---- GGUF block expansion (one super-block per call) ----
void deq_q4_0(const uint8_t* b, float* y) {  // 18 bytes -> 32 values
  const float d = half_to_float(rd<uint16_t>(b));
  const uint8_t* qs = b + 2;
  for (int j = 0; j < 16; ++j) {
    y[j] = static_cast<float>((qs[j] & 0x0F) - 8) * d;
    y[j + 16] = static_cast<float>((qs[j] >> 4) - 8) * d;
  }
}
void deq_q8_0(const uint8_t* b, float* y) {  // 34 bytes -> 32 values
  const float d = half_to_float(rd<uint16_t>(b));
  const int8_t* qs = reinterpret_cast<const int8_t*>(b + 2);
  for (int j = 0; j < 32; ++j) y[j] = static_cast<float>(qs[j]) * d;
}
inline void scale_min_k4(int j, const uint8_t* q, uint8_t* d, uint8_t* m) {
  if (j < 4) {
    *d = q[j] & 63;
    *m = q[j + 4] & 63;
  } else {
    *d = (q[j + 4] & 0xF) | ((q[j - 4] >> 6) << 4);
    *m = (q[j + 4] >> 4) | ((q[j] >> 6) << 4);
  }
}
void deq_q4_k(const uint8_t* b, float* y) {  // 144 bytes -> 256 values
  const float d = half_to_float(rd<uint16_t>(b));
  const float dmin = half_to_float(rd<uint16_t>(b + 2));
  const uint8_t* scales = b + 4;
  const uint8_t* q = b + 16;
  int is = 0;
  for (int j = 0; j < 256; j += 64) {
    uint8_t sc, m;
    scale_min_k4(is + 0, scales, &sc, &m);
    const float d1 = d * sc, m1 = dmin * m;
    scale_min_k4(is + 1, scales, &sc, &m);
    const float d2 = d * sc, m2 = dmin * m;
    for (int l = 0; l < 32; ++l) *y++ = d1 * (q[l] & 0xF) - m1;
    for (int l = 0; l < 32; ++l) *y++ = d2 * (q[l] >> 4) - m2;
    q += 32;
    is += 2;
  }
}
void deq_q6_k(const uint8_t* b, float* y) {  // 210 bytes -> 256 values
  const uint8_t* ql = b;
  const uint8_t* qh = b + 128;
  const int8_t* sc = reinterpret_cast<const int8_t*>(b + 192);
  const float d = half_to_float(rd<uint16_t>(b + 208));
  for (int n = 0; n < 256; n += 128) {
    for (int l = 0; l < 32; ++l) {
      const int is = l / 16;
      const int q1 = static_cast<int8_t>((ql[l + 0] & 0xF) | (((qh[l] >> 0) & 3) << 4)) - 32;
      const int q2 = static_cast<int8_t>((ql[l + 32] & 0xF) | (((qh[l] >> 2) & 3) << 4)) - 32;
      const int q3 = static_cast<int8_t>((ql[l + 0] >> 4) | (((qh[l] >> 4) & 3) << 4)) - 32;
      const int q4 = static_cast<int8_t>((ql[l + 32] >> 4) | (((qh[l] >> 6) & 3) << 4)) - 32;
      y[l + 0] = d * sc[is + 0] * q1;
      y[l + 32] = d * sc[is + 2] * q2;
      y[l + 64] = d * sc[is + 4] * q3;
      y[l + 96] = d * sc[is + 6] * q4;
    }
    y += 128;
    ql += 64;
    qh += 32;
    sc += 8;
  }
}

struct BlockFmt {
  int bytes, elems;
  void (*fn)(const uint8_t*, float*);
};
bool block_fmt(int32_t dtype, BlockFmt* f) {
  switch (dtype) {
    case kGGUF_Q4_0: *f = {18, 32, deq_q4_0}; return true;
    case kGGUF_Q8_0: *f = {34, 32, deq_q8_0}; return true;
    case kGGUF_Q4_K: *f = {144, 256, deq_q4_k}; return true;
    case kGGUF_Q6_K: *f = {210, 256, deq_q6_k}; return true;
    default: return false;
  }
}

}  // namespace

MllmFile::MllmFile(const std::string& path) {
  fd_ = ::open(path.c_str(), O_RDONLY);
  if (fd_ < 0) throw std::runtime_error("cannot open " + path);
  struct stat st;
  if (::fstat(fd_, &st) != 0 || st.st_size < 12) {
    ::close(fd_);
    throw std::runtime_error("cannot stat or file too small: " + path);
  }
  size_ = static_cast<uint64_t>(st.st_size);
  void* m = ::mmap(nullptr, size_, PROT_READ, MAP_PRIVATE, fd_, 0);
  if (m == MAP_FAILED) {
    ::close(fd_);
    throw std::runtime_error("mmap failed: " + path);
  }
  base_ = static_cast<const uint8_t*>(m);
  const int32_t magic = rd<int32_t>(base_);
  try {
    if (magic == kMagicV1) {
      parse_v1();
    } else if (magic == kMagicV2) {
      parse_v2();
    } else {
      throw std::runtime_error("not a .mllm file (bad magic): " + path);
    }
  } catch (...) {
    ::munmap(const_cast<uint8_t*>(base_), size_);
    ::close(fd_);
    throw;
  }
}

MllmFile::~MllmFile() {
  if (base_ != nullptr) ::munmap(const_cast<uint8_t*>(base_), size_);
  if (fd_ >= 0) ::close(fd_);
}

void MllmFile::parse_v1() {
  version_ = 1;
  const uint64_t table_len = rd<uint64_t>(base_ + 4);
  uint64_t pos = 12;
  const uint64_t end = 12 + table_len;
  if (end > size_) throw std::runtime_error(".mllm v1: descriptor table exceeds the file");
  while (pos < end) {
    if (pos + 4 > end) throw std::runtime_error(".mllm v1: truncated descriptor");
    const int32_t name_len = rd<int32_t>(base_ + pos);
    pos += 4;
    if (name_len < 0 || pos + static_cast<uint64_t>(name_len) + 20 > end) throw std::runtime_error(".mllm v1: bad name length");
    MllmParam p;
    p.name.assign(reinterpret_cast<const char*>(base_ + pos), static_cast<size_t>(name_len));
    pos += static_cast<uint64_t>(name_len);
    p.size = rd<uint64_t>(base_ + pos);
    p.offset = rd<uint64_t>(base_ + pos + 8);
    p.dtype = rd<int32_t>(base_ + pos + 16);
    pos += 20;
    if (p.offset + p.size > size_) throw std::runtime_error(".mllm v1: tensor " + p.name + " exceeds the file");
    params_.push_back(std::move(p));
  }
}

void MllmFile::parse_v2() {
  version_ = 2;
  if (size_ < kV2Header) throw std::runtime_error(".mllm v2: truncated header");
  const int32_t ver = rd<int32_t>(base_ + 4);
  if (ver != 2) throw std::runtime_error(".mllm v2: unsupported version");
  const char* nm = reinterpret_cast<const char*>(base_ + 8);
  model_name_.assign(nm, strnlen(nm, 512));
  const uint32_t n = rd<uint32_t>(base_ + 520);
  const uint64_t desc = rd<uint64_t>(base_ + 524);
  if (desc + static_cast<uint64_t>(n) * kV2Desc > size_) throw std::runtime_error(".mllm v2: descriptors exceed the file");
  params_.reserve(n);
  for (uint32_t i = 0; i < n; ++i) {
    const uint8_t* d = base_ + desc + static_cast<uint64_t>(i) * kV2Desc;
    MllmParam p;
    p.dtype = static_cast<int32_t>(rd<uint32_t>(d + 4));
    p.size = rd<uint64_t>(d + 8);
    p.offset = rd<uint64_t>(d + 16);
    const uint64_t rank = rd<uint64_t>(d + 24);
    if (rank > 16) throw std::runtime_error(".mllm v2: rank > 16");
    for (uint64_t r = 0; r < rank; ++r) p.shape.push_back(rd<int32_t>(d + 32 + 4 * r));
    const char* name = reinterpret_cast<const char*>(d + 96);
    p.name.assign(name, strnlen(name, 256));
    if (p.offset + p.size > size_) throw std::runtime_error(".mllm v2: tensor " + p.name + " exceeds the file");
    params_.push_back(std::move(p));
  }
}

const MllmParam* MllmFile::find(const std::string& name) const {
  for (const auto& p : params_)
    if (p.name == name) return &p;
  return nullptr;
}

int64_t gguf_num_elements(int32_t dtype, uint64_t bytes) {
  BlockFmt f;
  if (!block_fmt(dtype, &f) || bytes % f.bytes != 0) return 0;
  return static_cast<int64_t>(bytes / f.bytes) * f.elems;
}

bool gguf_dequantize(int32_t dtype, const uint8_t* src, uint64_t bytes, float* dst, int threads) {
  BlockFmt f;
  if (!block_fmt(dtype, &f) || bytes % f.bytes != 0) return false;
  const int64_t blocks = static_cast<int64_t>(bytes / f.bytes);
  int nt = threads > 0 ? threads : static_cast<int>(std::thread::hardware_concurrency());
  nt = static_cast<int>(std::max<int64_t>(1, std::min<int64_t>(nt, blocks / 1024 + 1)));
  auto work = [&](int64_t b0, int64_t b1) {
    for (int64_t b = b0; b < b1; ++b) f.fn(src + b * f.bytes, dst + b * f.elems);
  };
  if (nt == 1) {
    work(0, blocks);
    return true;
  }
  std::vector<std::thread> pool;
  for (int t = 0; t < nt; ++t) pool.emplace_back(work, blocks * t / nt, blocks * (t + 1) / nt);
  for (auto& th : pool) th.join();
  return true;
}

void write_mllm_v2(const std::string& path, const std::string& model_name, const std::vector<MllmWriteEntry>& entries) {
  std::ofstream out(path, std::ios::binary | std::ios::trunc);
  if (!out) throw std::runtime_error("cannot create " + path);
  std::vector<uint8_t> header(kV2Header, 0);
  const int32_t magic = kMagicV2, ver = 2;
  std::memcpy(header.data(), &magic, 4);
  std::memcpy(header.data() + 4, &ver, 4);
  std::memcpy(header.data() + 8, model_name.data(), std::min<size_t>(model_name.size(), 511));
  const uint32_t n = static_cast<uint32_t>(entries.size());
  const uint64_t desc_off = kV2Header;
  std::memcpy(header.data() + 520, &n, 4);
  std::memcpy(header.data() + 524, &desc_off, 8);
  out.write(reinterpret_cast<const char*>(header.data()), header.size());
  uint64_t data_off = (kV2Header + static_cast<uint64_t>(n) * kV2Desc + 63) / 64 * 64;
  std::vector<uint64_t> offsets;
  for (uint32_t i = 0; i < n; ++i) {
    const auto& e = entries[i];
    if (e.shape.size() > 16) throw std::runtime_error("write_mllm_v2: rank > 16 for " + e.name);
    if (e.name.size() > 255) throw std::runtime_error("write_mllm_v2: name longer than 255 bytes: " + e.name);
    std::vector<uint8_t> d(kV2Desc, 0);
    const uint32_t dt = static_cast<uint32_t>(e.dtype);
    const uint64_t rank = e.shape.size();
    std::memcpy(d.data(), &i, 4);
    std::memcpy(d.data() + 4, &dt, 4);
    std::memcpy(d.data() + 8, &e.size, 8);
    std::memcpy(d.data() + 16, &data_off, 8);
    std::memcpy(d.data() + 24, &rank, 8);
    for (uint64_t r = 0; r < rank; ++r) std::memcpy(d.data() + 32 + 4 * r, &e.shape[r], 4);
    std::memcpy(d.data() + 96, e.name.data(), e.name.size());
    out.write(reinterpret_cast<const char*>(d.data()), d.size());
    offsets.push_back(data_off);
    data_off = (data_off + e.size + 63) / 64 * 64;
  }
  uint64_t pos = kV2Header + static_cast<uint64_t>(n) * kV2Desc;
  const std::vector<char> zeros(64, 0);
  for (uint32_t i = 0; i < n; ++i) {
    if (offsets[i] > pos) out.write(zeros.data(), static_cast<std::streamsize>(offsets[i] - pos));
    out.write(reinterpret_cast<const char*>(entries[i].data), static_cast<std::streamsize>(entries[i].size));
    pos = offsets[i] + entries[i].size;
  }
  if (!out) throw std::runtime_error("write failed: " + path);
}

}  // namespace mb200host
