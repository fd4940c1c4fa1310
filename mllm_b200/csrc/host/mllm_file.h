// Reader / writer of the `.mllm` parameter container (versions 1 and 2) used by the mllm C++ runtime.
//
// V1: int32 magic 20012, uint64 descriptor-table length, then per parameter
//     {int32 name_len, name, uint64 data_len, uint64 offset, int32 dtype}; no shapes.
// V2: 532-byte header {int32 magic 0x519A, int32 version 2, char model_name[512], uint32 num_params,
//     uint64 params_desc_offset}, then num_params 352-byte descriptors {uint32 id, uint32 dtype,
//     uint64 size, uint64 offset, uint64 shape_len, int32 shape[16], char name[256]}, then data.
// The file is memory-mapped; tensors are handed out as views.  GGUF block formats
// (Q4_0, Q8_0, Q4_K, Q6_K) can be expanded to fp32 with a pool of threads.
#pragma once
#include <cstdint>
#include <string>
#include <vector>

namespace mb200host {

enum MllmDType : int32_t {
  kFloat32 = 0, kFloat16 = 1, kGGUF_Q4_0 = 2, kGGUF_Q8_0 = 8, kGGUF_Q4_K = 12, kGGUF_Q6_K = 14,
  kInt8 = 16, kInt16 = 17, kInt32 = 18, kBFloat16 = 128, kUInt8 = 129, kUInt16 = 130, kUInt32 = 131,
  kInt64 = 132, kUInt64 = 133, kByte = 134,
};

struct MllmParam {
  std::string name;
  int32_t dtype = 0;
  uint64_t size = 0;    // bytes
  uint64_t offset = 0;  // from the start of the file
  std::vector<int32_t> shape;  // empty for V1
};

class MllmFile {
 public:
  explicit MllmFile(const std::string& path);
  ~MllmFile();
  MllmFile(const MllmFile&) = delete;
  MllmFile& operator=(const MllmFile&) = delete;
  int version() const { return version_; }
  const std::string& model_name() const { return model_name_; }
  const std::vector<MllmParam>& params() const { return params_; }
  const MllmParam* find(const std::string& name) const;
  const uint8_t* data(const MllmParam& p) const { return base_ + p.offset; }
  uint64_t file_size() const { return size_; }

 private:
  void parse_v1();
  void parse_v2();
  int fd_ = -1;
  const uint8_t* base_ = nullptr;
  uint64_t size_ = 0;
  int version_ = 0;
  std::string model_name_;
  std::vector<MllmParam> params_;
};

// Elements stored in `bytes` bytes of a GGUF block format (0 for other dtypes).
int64_t gguf_num_elements(int32_t dtype, uint64_t bytes);
// Expands GGUF blocks to fp32; returns false for an unsupported dtype.  `threads` <= 0: hardware count.
bool gguf_dequantize(int32_t dtype, const uint8_t* src, uint64_t bytes, float* dst, int threads);

struct MllmWriteEntry {
  std::string name;
  int32_t dtype;
  std::vector<int32_t> shape;
  const uint8_t* data;
  uint64_t size;
};
// Writes a V2 file; data blocks are 64-byte aligned.
void write_mllm_v2(const std::string& path, const std::string& model_name, const std::vector<MllmWriteEntry>& entries);

}  // namespace mb200host
