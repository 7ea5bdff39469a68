/* Scaffolding that lets a few self-contained functions of the reference compile on their
 * own.  TEST INFRASTRUCTURE ONLY.  The function bodies themselves are never stored here:
 * the Makefile streams them from the reference tree into the compiler. */
#include <cmath>
#include <cstdint>
#include <cstring>
#include <vector>
typedef uint16_t bf16_t;
struct ModelConfig {
  int rope_dim = 64;
  std::vector<int> compress_ratios;
};
class FSTEngine {
 public:
  ModelConfig config_;
  float rope_freq_base_ = 10000.0f;
  int seq_pos_ = 0;
  void build_rope_lut(bf16_t* lut, int M, int lid, bool inverse = false);
};
