// FSTEngine (MLA subset) over the CUDA C ABI.  See fst_engine.h.
#include "fst_engine.h"
#include "fst_file.h"

#include <cmath>
#include <cstring>
#include <stdexcept>

static inline float bf16f(bf16_t v) {  // reference src/fst_engine.cpp:26
  uint32_t b = (uint32_t)v << 16;
  float f;
  memcpy(&f, &b, 4);
  return f;
}
static inline bf16_t f2bf(float f) {  // reference src/fst_engine.cpp:27 (truncating)
  uint32_t b;
  memcpy(&b, &f, 4);
  return (bf16_t)(b >> 16);
}

void FSTEngine::check(int rc, const char* what) {
  if (rc != FST_MLA_OK)
    throw std::runtime_error(std::string(what) + ": " + fst_cuda_mla_last_error());
}

FSTEngine::FSTEngine(const ModelConfig& cfg) : config_(cfg) {
  shared_.resize(cfg.n_layers);
  FstMlaConfig c;
  memset(&c, 0, sizeof(c));
  c.preset = cfg.preset;
  c.hidden = cfg.hidden_dim;
  c.n_heads = MLA_N_HEADS;
  c.q_lora = MLA_Q_LORA;
  c.kv_lora = MLA_KV_LORA;
  c.qk_nope = 128;
  c.qk_rope = cfg.rope_dim;
  c.v_head = 128;
  c.o_groups = 8;
  c.o_lora = 1024;
  c.rope_theta = cfg.rope_freq_base > 0.0f ? cfg.rope_freq_base : 10000.0f;
  c.rms_eps = 1e-6f;
  c.rope_yarn = 0;  // the kind is a property of each layer: preload_all_layers sets it
  c.n_layers = cfg.n_layers;
  c.page_tokens = cfg.page_tokens;
  const int pages_per_seq = (cfg.max_seq + cfg.page_tokens - 1) / cfg.page_tokens;
  // the rows of a sequence, plus (V4 form) its compressed rows: at most one per four rows, in
  // pages of their own
  const int cmp_pages_per_seq = cfg.preset == FST_MLA_PRESET_FASTAR_V4
                                    ? (cfg.max_seq / 4 + cfg.page_tokens - 1) / cfg.page_tokens : 0;
  c.n_pages = (pages_per_seq + cmp_pages_per_seq) * cfg.max_seqs;
  c.max_seqs = cfg.max_seqs;
  c.max_tokens = cfg.max_tokens;
  c.device = cfg.device;
  c.attn_impl = cfg.attn_impl;
  c.gemm_impl = cfg.gemm_impl;
  check(fst_cuda_mla_create(&c, &ctx_), "fst_cuda_mla_create");
  int32_t s = -1;
  check(fst_cuda_mla_seq_alloc(ctx_, &s), "seq_alloc");
  seq_ = s;
}

FSTEngine::~FSTEngine() { fst_cuda_mla_destroy(ctx_); }

namespace {

// expected element counts of the MLA tensors of one layer, by preset
struct MlaSizes {
  size_t wq_a, wq_b, wkv, wo_a, wo_b, q_norm, kv_norm, sinks, attn_norm;
};

MlaSizes sizes_of(const ModelConfig& c) {
  const size_t hd = (size_t)c.hidden_dim, H = MLA_N_HEADS, low = 8192;
  MlaSizes z;
  z.wq_a = (size_t)MLA_Q_LORA * hd;
  z.q_norm = MLA_Q_LORA;
  z.kv_norm = MLA_KV_LORA;
  z.sinks = H;
  z.attn_norm = hd;
  z.wo_b = hd * low;
  if (c.preset == FST_MLA_PRESET_FASTAR_V4) {
    z.wq_b = H * (size_t)MLA_HEAD_DIM * MLA_Q_LORA;
    z.wkv = (size_t)MLA_KV_LORA * hd;
    z.wo_a = low * (H * (size_t)MLA_HEAD_DIM / 8);
  } else {
    z.wq_b = H * 192 * (size_t)MLA_Q_LORA;
    z.wkv = (size_t)(MLA_KV_LORA + MLA_ROPE_DIM) * hd;
    z.wo_a = 0;  // the BASELINE form has no wo_a (W_UV comes with wkv_b, which the file format does not carry)
  }
  return z;
}

// A matrix is looked up by its shape among the entries of its tensor id first, as the engine finds
// it (src/fst_engine.cpp:1553-1558, 1610-1615) -- one converter path stores wq_a / wq_b and wo_a / wo_b
// under one (tensor id, sub id) -- and by its sub id when no entry has the expected shape.
void take_bf16(const std::string& path, const std::vector<fstfile::Entry>& dir, uint32_t tid, int layer, int sub,
               size_t want, const char* name, std::vector<bf16_t>* dst, uint64_t rows = 0, uint64_t cols = 0) {
  const fstfile::Entry* e = rows ? fstfile::find_shape(dir, tid, layer, rows, cols ? cols : 1) : nullptr;
  if (!e) e = fstfile::find(dir, tid, layer, sub);
  if (!e) return;
  std::vector<uint16_t> v = fstfile::load_bf16(path, *e);
  if (want && v.size() != want)
    throw std::runtime_error(path + ": layer " + std::to_string(layer) + " " + name + " has " + std::to_string(v.size()) +
                             " values, the configuration wants " + std::to_string(want));
  dst->assign(v.begin(), v.end());
}

void take_sinks(const std::string& path, const std::vector<fstfile::Entry>& dir, int layer, size_t want,
                std::vector<float>* dst) {
  const fstfile::Entry* e = fstfile::find(dir, fstfile::TID_ATTN_SINK, layer, 0);
  if (!e) return;
  std::vector<float> v = fstfile::load_f32(path, *e);
  if (v.size() < want)
    throw std::runtime_error(path + ": layer " + std::to_string(layer) + " attn_sinks has " + std::to_string(v.size()) + " values");
  dst->assign(v.begin(), v.begin() + want);  // the engine copies the first n_heads (src/fst_engine.cpp:1630-1636)
}

}  // namespace

bool FSTEngine::layer_is_compressed(int lid) const {
  if (config_.preset != FST_MLA_PRESET_FASTAR_V4) return false;
  return lid < (int)config_.compress_ratios.size() ? config_.compress_ratios[lid] != 0 : lid >= 2;
}

void FSTEngine::load_shared_weights(const std::string& fst_path) {
  fstfile::Header hd;
  const std::vector<fstfile::Entry> dir = fstfile::read_directory(fst_path, &hd);
  const MlaSizes z = sizes_of(config_);
  // rope_freq_base_ comes from the header (src/fst_engine.cpp:1505)
  config_.rope_freq_base = hd.rope_freq_base;
  check(fst_cuda_mla_set_rope_theta(ctx_, config_.rope_freq_base), "set_rope_theta");
  // compress_ratios: TID 40, F32 [n_layers], float -> int; without it the default pattern 0, 0, 4,
  // 128, 4, ... with the last two layers uncompressed from layer 41 on (1559-1590)
  config_.compress_ratios.assign(config_.n_layers, 0);
  const fstfile::Entry* cr = nullptr;
  for (const fstfile::Entry& e : dir)
    if (e.tid == fstfile::TID_COMPRESS_RATIOS) {
      cr = &e;
      break;
    }
  if (cr) {
    const std::vector<float> r = fstfile::load_f32(fst_path, *cr);
    for (int l = 0; l < config_.n_layers && l < (int)r.size(); ++l) config_.compress_ratios[l] = (int)r[l];
  } else {
    for (int l = 0; l < config_.n_layers; ++l) config_.compress_ratios[l] = (l < 2 || l >= 41) ? 0 : (l % 2 == 0 ? 4 : 128);
  }
  const uint64_t hdim = (uint64_t)config_.hidden_dim, low = 8192;
  const bool v4 = config_.preset == FST_MLA_PRESET_FASTAR_V4;
  for (int l = 0; l < config_.n_layers; ++l) {
    LayerWeightsC& w = shared_.at(l);
    take_bf16(fst_path, dir, fstfile::TID_Q_PROJ, l, 0, z.wq_a, "wq_a", &w.wq_a, MLA_Q_LORA, hdim);
    take_bf16(fst_path, dir, fstfile::TID_Q_PROJ, l, 1, z.wq_b, "wq_b", &w.wq_b, z.wq_b / MLA_Q_LORA, MLA_Q_LORA);
    take_bf16(fst_path, dir, fstfile::TID_K_PROJ, l, 0, z.wkv, "wkv", &w.wkv);
    if (v4) take_bf16(fst_path, dir, fstfile::TID_O_PROJ, l, 0, z.wo_a, "wo_a", &w.wo_a, low, z.wo_a / low);
    take_bf16(fst_path, dir, fstfile::TID_O_PROJ, l, 1, z.wo_b, "wo_b", &w.wo_b, hdim, low);
    take_bf16(fst_path, dir, fstfile::TID_Q_NORM, l, 0, z.q_norm, "q_norm", &w.q_norm);
    take_bf16(fst_path, dir, fstfile::TID_KV_NORM, l, 0, z.kv_norm, "kv_norm", &w.kv_norm);
    take_bf16(fst_path, dir, fstfile::TID_INPUT_NORM, l, 0, z.attn_norm, "attn_norm", &w.attn_norm);
    take_sinks(fst_path, dir, l, z.sinks, &w.attn_sinks);
    // V4 KV compressor weights, TIDs 32-35, only for layers with a ratio (1657-1690)
    w.cmp_ratio = v4 && l < (int)config_.compress_ratios.size() ? config_.compress_ratios[l] : 0;
    w.cmp_comp_width = w.cmp_ratio == 4 ? 2 * MLA_KV_LORA : (w.cmp_ratio == 128 ? MLA_KV_LORA : 0);
    if (w.cmp_comp_width) {
      const size_t cw = (size_t)w.cmp_comp_width;
      if (const fstfile::Entry* e = fstfile::find(dir, 32, l, 0)) {
        std::vector<float> ape = fstfile::load_f32(fst_path, *e);
        if (ape.size() >= (size_t)w.cmp_ratio * cw) w.cmp_ape.assign(ape.begin(), ape.begin() + (size_t)w.cmp_ratio * cw);
      }
      take_bf16(fst_path, dir, 33, l, 0, cw * hdim, "cmp_wkv", &w.cmp_wkv);
      take_bf16(fst_path, dir, 34, l, 0, cw * hdim, "cmp_wgate", &w.cmp_wgate);
      take_bf16(fst_path, dir, 35, l, 0, MLA_KV_LORA, "cmp_norm", &w.cmp_norm);
    }
  }
}

void FSTEngine::load_norm_override(const std::string& norm_path) {
  const std::vector<fstfile::Entry> dir = fstfile::read_directory(norm_path);
  const MlaSizes z = sizes_of(config_);
  for (int l = 0; l < config_.n_layers; ++l) {
    LayerWeightsC& w = shared_.at(l);
    take_bf16(norm_path, dir, fstfile::TID_INPUT_NORM, l, 0, z.attn_norm, "attn_norm", &w.attn_norm);
    take_bf16(norm_path, dir, fstfile::TID_Q_NORM, l, 0, z.q_norm, "q_norm", &w.q_norm);
    take_bf16(norm_path, dir, fstfile::TID_KV_NORM, l, 0, z.kv_norm, "kv_norm", &w.kv_norm);
    take_sinks(norm_path, dir, l, z.sinks, &w.attn_sinks);
  }
}

void FSTEngine::preload_all_layers() {
  for (int l = 0; l < config_.n_layers; ++l) {
    const LayerWeightsC& w = shared_[l];
    FstMlaWeights fw;
    memset(&fw, 0, sizeof(fw));
    auto p = [](const std::vector<bf16_t>& v) { return v.empty() ? nullptr : v.data(); };
    fw.wq_a = p(w.wq_a);
    fw.wq_b = p(w.wq_b);
    fw.wkv_a = p(w.wkv);
    fw.wkv_b = p(w.wkv_b);
    fw.wo_a = p(w.wo_a);
    fw.wo_b = p(w.wo_b);
    fw.q_norm = p(w.q_norm);
    fw.kv_norm = p(w.kv_norm);
    fw.attn_sinks = w.attn_sinks.empty() ? nullptr : w.attn_sinks.data();
    fw.attn_norm = p(w.attn_norm);
    check(fst_cuda_mla_set_layer_weights(ctx_, l, &fw), "set_layer_weights");
    check(fst_cuda_mla_set_layer_rope(ctx_, l, layer_is_compressed(l) ? 1 : 0), "set_layer_rope");
    if (config_.draft) check(fst_cuda_mla_set_layer_draft_form(ctx_, l, 1), "set_layer_draft_form");
    if (use_compressor_ && w.cmp_ratio != 0 && !w.cmp_wkv.empty() && !w.cmp_wgate.empty() && !w.cmp_ape.empty() &&
        !w.cmp_norm.empty()) {  // (the conditions of compress_token, 3173-3175)
      FstMlaCompressor cw;
      cw.ratio = w.cmp_ratio;
      cw.wkv = w.cmp_wkv.data();
      cw.wgate = w.cmp_wgate.data();
      cw.ape = w.cmp_ape.data();
      cw.norm = w.cmp_norm.data();
      check(fst_cuda_mla_set_layer_compressor(ctx_, l, &cw), "set_layer_compressor");
    }
  }
}

void FSTEngine::process_mla(int lid, bf16_t* h, int M) {
  if (seq_pos_ + M > config_.max_seq)  // assert(seq_pos_ + M <= config_.max_seq), reference 3327
    throw std::runtime_error("process_mla: seq_pos_ + M exceeds max_seq");
  const int32_t seq = seq_, pos = seq_pos_, q = M;
  check(fst_cuda_mla_forward(ctx_, lid, h, h, &seq, &pos, &q, 1, is_prefill_ ? 1 : 0), "process_mla");
}

void FSTEngine::process_draft_mla(int lid, bf16_t* h, int M, const bf16_t* main_x) {
  const int anchor = seq_pos_;
  if (anchor + 1 + M > config_.max_seq) throw std::runtime_error("process_draft_mla: anchor + 1 + M exceeds max_seq");
  const int32_t seq = seq_, one = 1;
  int32_t pos = anchor, q = M;
  // main_kv = kv_norm(wkv(main_x)), rotary at the anchor, into the window (4913-4940)
  check(fst_cuda_mla_append_rows(ctx_, lid, main_x, &seq, &pos, &one, 1), "process_draft_mla (main row)");
  // q and kv of the block at anchor+1+m, dense attention over [window ; block] with the sink, inverse
  // rotation, grouped wo_a, wo_b (4942-5131).  The ring of window_size slots becomes a window on the
  // paged rows: the last window_size main rows and the M block rows.
  const int win = config_.window_size;
  check(fst_cuda_mla_set_window(ctx_, anchor + 1 > win ? win + M : 0), "set_window");
  pos = anchor + 1;
  check(fst_cuda_mla_forward(ctx_, lid, h, h, &seq, &pos, &q, 1, 0), "process_draft_mla");
  check(fst_cuda_mla_set_window(ctx_, 0), "set_window");
  // only main rows stay in the cache: the block's rows go again
  check(fst_cuda_mla_seq_truncate(ctx_, seq_, anchor + 1), "process_draft_mla (drop the block)");
}

void FSTEngine::process_mla_batch(int lid, bf16_t* h, const int* seq_ids, const int* pos0, const int* q_lens, int B,
                                  bool causal) {
  for (int b = 0; b < B; ++b)
    if (pos0[b] + q_lens[b] > config_.max_seq) throw std::runtime_error("process_mla_batch: a sequence exceeds max_seq");
  check(fst_cuda_mla_forward(ctx_, lid, h, h, seq_ids, pos0, q_lens, B, causal ? 1 : 0), "process_mla_batch");
}

void FSTEngine::join_split_group(const uint8_t id[128], int rank, int world) {
  check(fst_cuda_mla_comm_init(ctx_, id, rank, world), "comm_init");
}

void FSTEngine::process_mla_split(int lid, bf16_t* h, int M, bool owns_new_rows) {
  int32_t local_len = 0;
  check(fst_cuda_mla_seq_len(ctx_, seq_, &local_len), "seq_len");
  FstMlaSeqStep st;
  st.seq = seq_;
  st.pos0 = owns_new_rows ? seq_pos_ - slice_begin_ : local_len;  // local row of the first new token / rows held
  st.q_len = M;
  st.rope_pos0 = seq_pos_;  // RoPE uses the global position
  st.append = owns_new_rows ? 1 : 0;
  st.window = 0;
  if (owns_new_rows && st.pos0 + M > config_.max_seq) throw std::runtime_error("process_mla_split: the slice exceeds max_seq");
  check(fst_cuda_mla_forward_split(ctx_, lid, h, h, &st, 1, 0), "process_mla_split");
}

void FSTEngine::reset_session() {
  check(fst_cuda_mla_reset(ctx_), "reset");
  int32_t s = -1;
  check(fst_cuda_mla_seq_alloc(ctx_, &s), "seq_alloc");
  seq_ = s;
  seq_pos_ = 0;
  is_prefill_ = true;
}

void FSTEngine::set_window(int window) { check(fst_cuda_mla_set_window(ctx_, window), "set_window"); }

void FSTEngine::snapshot_before_verify() { check(fst_cuda_mla_seq_snapshot(ctx_, seq_), "seq_snapshot"); }

void FSTEngine::rollback(int keep_len) {
  int32_t len = 0;
  check(fst_cuda_mla_seq_len(ctx_, seq_, &len), "seq_len");
  if (keep_len < len) check(fst_cuda_mla_seq_truncate(ctx_, seq_, keep_len), "seq_truncate");
  seq_pos_ = keep_len;
}

int FSTEngine::new_sequence() {
  int32_t s = -1;
  check(fst_cuda_mla_seq_alloc(ctx_, &s), "seq_alloc");
  return s;
}

void FSTEngine::free_sequence(int seq) { check(fst_cuda_mla_seq_free(ctx_, seq), "seq_free"); }

std::vector<RandmatResult> FSTEngine::randmat_test() {
  // same generator, shapes and reference computation as the engine's probe (592-640)
  uint64_t st = 0x123456789abcdefULL;
  auto nxt = [&]() -> uint32_t {
    st ^= st << 13;
    st ^= st >> 7;
    st ^= st << 17;
    return (uint32_t)(st >> 32);
  };
  auto rbf = [&]() -> bf16_t { return f2bf(((float)(nxt() & 0xffff) / 65535.0f) * 2.0f - 1.0f); };
  struct Probe { const char* name; int K, N; };
  const Probe probes[] = {{"ffn_gate/up", 4096, 2048}, {"ffn_down", 2048, 2048}, {"qc (wq_a)", 4096, 1024},
                          {"wqb (wq_b)", 1024, 2048},  {"ob (wo_b)", 8192, 2048}, {"qck (full K)", 4096, 1024}};
  const int M = 16;
  std::vector<RandmatResult> out;
  for (const auto& p : probes) {
    std::vector<bf16_t> A((size_t)M * p.K), B((size_t)p.N * p.K), C((size_t)M * p.N, 0);
    for (auto& v : A) v = rbf();
    for (auto& v : B) v = rbf();
    check(fst_cuda_mla_gemm(ctx_, C.data(), A.data(), B.data(), M, p.N, p.K, 0), "gemm");
    double dot = 0, nn = 0, nr = 0, me = 0;
    for (int m = 0; m < M; ++m)
      for (int n = 0; n < p.N; ++n) {
        double acc = 0;
        for (int k = 0; k < p.K; ++k) acc += (double)bf16f(A[(size_t)m * p.K + k]) * (double)bf16f(B[(size_t)n * p.K + k]);
        const double got = bf16f(C[(size_t)m * p.N + n]);
        dot += got * acc;
        nn += got * got;
        nr += acc * acc;
        me = std::max(me, std::fabs(got - acc));
      }
    out.push_back({p.name, M, p.K, p.N, dot / (std::sqrt(nn) * std::sqrt(nr) + 1e-30), std::sqrt(nn / nr), me});
  }
  return out;
}
