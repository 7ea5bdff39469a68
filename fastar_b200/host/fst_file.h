// Reader for the MLA tensors of a `.fst` checkpoint, host side (no device calls).
//
// File layout as the reference's converter writes it (scripts/fst_converter.py:173-176, 685-716,
// 1464-1500) and its engine reads it (src/fst_engine.cpp:1503-1642, 1873-1900): a 128-byte header,
// a directory of 64-byte entries (tensor id, layer, sub id, qtype, ndim, shape[3], offset, size)
// and page-aligned payloads in BF16 (qtype 2), F32 (3) or Q8_0 (1: all fp16 block scales first,
// then all int8 values, 32 per block).  Tensors are found by tensor id and sub id, the way the
// engine reads its `.norm` sidecar (1873-1900); Q8_0 expands as in load_shared_weights
// (1593-1597): value * scale, a zero scale read as 1, fp32 -> bf16 by truncation.
#pragma once
#include <cstdint>
#include <string>
#include <vector>

namespace fstfile {

constexpr uint32_t TID_INPUT_NORM = 3, TID_Q_PROJ = 5, TID_K_PROJ = 6, TID_O_PROJ = 8;
constexpr uint32_t TID_Q_NORM = 14, TID_KV_NORM = 15, TID_ATTN_SINK = 22;
constexpr uint32_t TID_COMPRESS_RATIOS = 40;  // F32 [n_layers], stored once (src/fst_engine.cpp:1559-1590)
constexpr int QTYPE_Q8_0 = 1, QTYPE_BF16 = 2, QTYPE_F32 = 3;
constexpr int GLOBAL_LAYER = 0xFFFF;

struct Header {
  uint32_t version = 0, hidden_dim = 0, n_layers = 0, n_experts = 0, top_k = 0, n_q_heads = 0, n_kv_heads = 0,
           head_dim = 0;
  uint64_t vocab_size = 0;
  float rms_eps = 0.0f, rope_freq_base = 10000.0f;
  uint64_t dir_offset = 0, dir_count = 0;
};

struct Entry {
  uint32_t tid = 0;
  int layer = 0, sub = 0, qtype = 0, ndim = 0;
  uint64_t shape[3] = {1, 1, 1};
  uint64_t offset = 0, size = 0;
  uint64_t n_elements() const;
};

// All three throw std::runtime_error with the file name and the reason.
Header read_header(const std::string& path);
std::vector<Entry> read_directory(const std::string& path, Header* header_out = nullptr);
// First entry with this tensor id and sub id for the layer (or stored as global); nullptr if none.
const Entry* find(const std::vector<Entry>& dir, uint32_t tid, int layer, int sub = 0);
// First entry with this tensor id for the layer (or global) whose shape is [s0, s1]: the engine itself
// finds its matrices by shape (src/fst_engine.cpp:1553-1558, 1610-1615), and one of the converter's
// paths stores wq_a and wq_b (and wo_a and wo_b) under the same tensor id AND sub id 0
// (scripts/fst_converter.py:636-644), so the sub id alone cannot tell them apart.
const Entry* find_shape(const std::vector<Entry>& dir, uint32_t tid, int layer, uint64_t s0, uint64_t s1);
// BF16 and Q8_0 tensors as bf16 bits; an F32 tensor is truncated to bf16.
std::vector<uint16_t> load_bf16(const std::string& path, const Entry& e);
// F32 tensors as they are; BF16 and Q8_0 widened to fp32.
std::vector<float> load_f32(const std::string& path, const Entry& e);

}  // namespace fstfile
