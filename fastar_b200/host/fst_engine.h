// Host side of the MLA path, shaped like the reference engine (include/fst_engine.h) so that
// process_mla is a drop-in: the same entry point, the same implicit state (seq_pos_,
// is_prefill_, shared_[lid]), the same in-place contract on `h`.  What changes underneath is
// what the reference did with NPU dispatches and XRT buffer objects: weights, the latent cache
// (now paged, device resident) and every intermediate live on the GPU behind the C ABI of
// include/fst_cuda_mla.h.  Only the MLA subset of the engine exists here; the MoE / expert
// pager / sampler / tokenizer sides are not part of this library.
#pragma once
#include <cstdint>
#include <string>
#include <vector>

#include "fst_cuda_mla.h"

typedef uint16_t bf16_t;  // reference include/fst_engine.h:16

// reference include/fst_engine.h:92-95
constexpr int MLA_Q_LORA = 1024, MLA_KV_LORA = 512;
constexpr int MLA_N_HEADS = 64, MLA_HEAD_DIM = 512, MLA_Q_FLAT = MLA_N_HEADS * MLA_HEAD_DIM;
constexpr int MLA_ROPE_DIM = 64;

// reference ModelConfig (include/fst_engine.h:127-139), MLA members plus the paged-cache sizes.
struct ModelConfig {
  int n_layers = 1;
  int hidden_dim = 4096;
  int max_seq = 128;        // capacity of one sequence (the reference's flat cache length)
  int rope_dim = MLA_ROPE_DIM;
  std::vector<int> compress_ratios;  // per layer; non-zero selects the YaRN RoPE table (1979-1982)
  float rope_freq_base = 10000.0f;   // base of the plain tables (rope_freq_base_, 1505: the file header's, else 10000)
  // what this build adds
  int preset = FST_MLA_PRESET_FASTAR_V4;  // FST_MLA_PRESET_BASELINE for the 576-wide form
  int page_tokens = 64;
  int max_seqs = 1;         // sequences alive at once (batched decode)
  int max_tokens = 16;      // new tokens per layer call (prefill_tiled feeds 16, src/fst_engine.cpp:2959)
  int device = 0;
  int attn_impl = FST_MLA_IMPL_AUTO;
  int gemm_impl = FST_MLA_IMPL_AUTO;
  // the draft model (reference draft_cfg_): its layers have the draft form of the attention and
  // keep window_size main rows (draft_cfg_.window_size, 128)
  bool draft = false;
  int window_size = 128;
};

// reference LayerWeightsC (include/fst_engine.h:165-188), MLA members; bf16 [N_out, K_in].
struct LayerWeightsC {
  std::vector<bf16_t> q_norm, kv_norm, wq_a, wq_b, wkv, wo_a, wo_b;
  std::vector<bf16_t> wkv_b;        // BASELINE preset: per head W_UK rows then W_UV rows
  std::vector<float> attn_sinks;    // per-head sink logit (empty: 0, src/fst_engine.cpp:3623)
  std::vector<bf16_t> attn_norm;    // [hidden]; when set, process_mla takes the rows BEFORE the norm
                                    // of process_layer (src/fst_engine.cpp:2687-2688) and applies it
  // V4 KV compressor (reference include/fst_engine.h:172-180): cmp_ape F32 [ratio, comp_width],
  // cmp_wkv / cmp_wgate BF16 [comp_width, hidden] native [N, K], cmp_norm BF16 [512]; empty for
  // ratio-0 layers.  cmp_ratio 4 | 128, cmp_comp_width 1024 | 512.
  std::vector<float> cmp_ape;
  std::vector<bf16_t> cmp_wkv, cmp_wgate, cmp_norm;
  int cmp_ratio = 0;
  int cmp_comp_width = 0;
};

struct RandmatResult {  // one line of randmat_test (src/fst_engine.cpp:586-685)
  std::string name;
  int M, K, N;
  double cosine, norm_ratio, max_abs_err;
};

class FSTEngine {
 public:
  ModelConfig config_;
  std::vector<LayerWeightsC> shared_;

  // The reference constructor loads a .fst file (src/fst_engine.cpp:1250); model loading is
  // outside this path, so the caller fills shared_ and calls preload_all_layers().
  explicit FSTEngine(const ModelConfig& cfg);
  ~FSTEngine();
  FSTEngine(const FSTEngine&) = delete;
  FSTEngine& operator=(const FSTEngine&) = delete;

  // The MLA tensors of every layer from a `.fst` file into shared_[*] (the MLA share of
  // load_shared_weights, src/fst_engine.cpp:1503-1642: wq_a, wq_b, wkv, wo_a, wo_b, q_norm, kv_norm,
  // attn_sinks, attn_norm; BF16 or Q8_0), and the norm weights and sinks of a `.norm` sidecar over
  // them (load_norm_override, 1873-1900).  Host only: call preload_all_layers() afterwards.
  // Tensors the file does not hold stay as they are; a tensor of the wrong size is an error.
  void load_shared_weights(const std::string& fst_path);
  void load_norm_override(const std::string& norm_path);

  // Upload shared_[*] to the device (preload_all_layers, src/fst_engine.cpp:1152-1197).
  void preload_all_layers();

  // The hot path (src/fst_engine.cpp:3320-3890): h[M, hidden] attn-normed rows at positions
  // seq_pos_ .. seq_pos_+M-1 of the current sequence, overwritten with the attention output.
  // Causal among the M rows when is_prefill_ (3626).  Throws std::runtime_error on failure;
  // seq_pos_ + M > max_seq is an error (the reference asserts, 3327).
  void process_mla(int lid, bf16_t* h, int M);

  // The draft model's attention (process_draft_mla, src/fst_engine.cpp:4884-5131): main_x[hidden] is
  // the projected main hidden row -- its KV row enters the cache at the anchor position seq_pos_ --
  // and h[M, hidden] is the block of candidates at positions seq_pos_+1 .. seq_pos_+M, which attend
  // (densely, no causal mask) to the last window_size main rows and to the whole block; h is
  // overwritten with the attention output, and the block's own rows are not kept.  The caller
  // advances seq_pos_ (forward_draft does, one anchor per accepted row).
  void process_draft_mla(int lid, bf16_t* h, int M, const bf16_t* main_x);

  // Batched sibling: B sequences, q_lens[b] new rows each at pos0[b]; h is [sum q_lens, hidden].
  void process_mla_batch(int lid, bf16_t* h, const int* seq_ids, const int* pos0, const int* q_lens, int B,
                         bool causal);

  // Session state (reset_session 2992-3012; seq_pos_ advanced by the caller, 2972 / 6262).
  void reset_session();
  int seq_pos() const { return seq_pos_; }
  void set_seq_pos(int p) { seq_pos_ = p; }
  void advance(int n) { seq_pos_ += n; }
  void set_prefill(bool p) { is_prefill_ = p; }
  bool is_prefill() const { return is_prefill_; }
  // Speculative-decoding rollback (6132-6152): forget rows >= keep_len of the current sequence.  The
  // reference saves the compressor state before a verify block (cmp_snap) and restores it with the
  // rollback: snapshot_before_verify() is that save, rollback() to the same length restores it.
  void snapshot_before_verify();
  void rollback(int keep_len);
  // The KV compressor runs for layers that carry its weights (the reference gates it behind the
  // FST_COMPRESSOR environment variable, 3565): off by default here too; call before preload_all_layers.
  void enable_compressor(bool on) { use_compressor_ = on; }
  // Sliding window of the draft model's attention (draft_cfg_.window_size, 2534-2576): process_mla
  // attends to the last `window` rows only; 0 switches it off.
  void set_window(int window);

  // One long sequence with its cache split along the KV axis over `world` engines, one per GPU
  // (the reference has no counterpart: one NPU, 128 rows).  This engine's cache holds the global
  // rows from slice_begin on; seq_pos_ stays the GLOBAL position.  join_split_group is collective
  // (ncclCommInitRank; id: the 128 bytes of fst_cuda_mla_comm_unique_id from rank 0).
  // process_mla_split: every engine computes the query, attends to its slice, one all-gather
  // exchanges the per-GPU partials, every engine merges and projects; `owns_new_rows` is true on the
  // engine whose slice the new rows extend.  Decode only (no causal block).
  void join_split_group(const uint8_t id[128], int rank, int world);
  void set_kv_slice(int slice_begin) { slice_begin_ = slice_begin; }
  void process_mla_split(int lid, bf16_t* h, int M, bool owns_new_rows);

  // Extra sequences for batched decode.
  int new_sequence();
  void free_sequence(int seq);
  int current_sequence() const { return seq_; }

  // Random-matrix probe of the GEMM tile engine (randmat_test, 586-685): xorshift-seeded
  // uniform [-1, 1] bf16 A[16, K], B[N, K] against a double-precision CPU product.
  std::vector<RandmatResult> randmat_test();

  // RoPE kind of a layer as build_rope_lut chooses it (src/fst_engine.cpp:1979-1982): YaRN when the
  // layer's compress ratio is non-zero; a layer the ratios do not cover counts as compressed from
  // layer 2 on.  The 576-wide BASELINE form has no compressed layers.
  bool layer_is_compressed(int lid) const;

  FstMlaCtx* ctx() { return ctx_; }

 private:
  FstMlaCtx* ctx_ = nullptr;
  int seq_ = -1;
  int seq_pos_ = 0;
  bool is_prefill_ = true;
  int slice_begin_ = 0;
  bool use_compressor_ = false;
  void check(int rc, const char* what);
};
