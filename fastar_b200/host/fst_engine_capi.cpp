// C entry points around FSTEngine so that the test harness can drive the C++ host class
// through ctypes.  Exceptions become return codes; the message is kept for the caller.
#include <cstring>
#include <stdexcept>
#include <string>

#include "fst_engine.h"
#include "fst_file.h"

namespace {
thread_local std::string g_msg;
template <class F>
int guard(F&& f) {
  try {
    f();
    return 0;
  } catch (const std::exception& e) {
    g_msg = e.what();
    return -1;
  }
}
}  // namespace

extern "C" {

const char* fst_engine_last_error() { return g_msg.c_str(); }

FSTEngine* fst_engine_create(int preset, int n_layers, int max_seq, int max_seqs, int max_tokens, int device,
                             int attn_impl, int gemm_impl) {
  FSTEngine* e = nullptr;
  guard([&] {
    ModelConfig c;
    c.preset = preset;
    c.n_layers = n_layers;
    c.max_seq = max_seq;
    c.max_seqs = max_seqs;
    c.max_tokens = max_tokens;
    c.device = device;
    c.attn_impl = attn_impl;
    c.gemm_impl = gemm_impl;
    e = new FSTEngine(c);
  });
  return e;
}
void fst_engine_destroy(FSTEngine* e) { delete e; }

// name: one of wq_a wq_b wkv wkv_b wo_a wo_b q_norm kv_norm attn_norm; n elements of bf16 bits.
int fst_engine_set_weight(FSTEngine* e, int lid, const char* name, const uint16_t* data, size_t n) {
  return guard([&] {
    LayerWeightsC& w = e->shared_.at(lid);
    std::vector<bf16_t>* dst = nullptr;
    const std::string s(name);
    if (s == "wq_a") dst = &w.wq_a;
    else if (s == "wq_b") dst = &w.wq_b;
    else if (s == "wkv" || s == "wkv_a") dst = &w.wkv;
    else if (s == "wkv_b") dst = &w.wkv_b;
    else if (s == "wo_a") dst = &w.wo_a;
    else if (s == "wo_b") dst = &w.wo_b;
    else if (s == "q_norm") dst = &w.q_norm;
    else if (s == "attn_norm") dst = &w.attn_norm;
    else if (s == "kv_norm") dst = &w.kv_norm;
    else throw std::runtime_error("unknown weight " + s);
    dst->assign(data, data + n);
  });
}
int fst_engine_set_sinks(FSTEngine* e, int lid, const float* data, size_t n) {
  return guard([&] { e->shared_.at(lid).attn_sinks.assign(data, data + n); });
}
int fst_engine_load_shared_weights(FSTEngine* e, const char* path) { return guard([&] { e->load_shared_weights(path); }); }
int fst_engine_load_norm_override(FSTEngine* e, const char* path) { return guard([&] { e->load_norm_override(path); }); }
// Host-only probe of the `.fst` reader (no engine, no device): the tensor (tid, layer, sub) as bf16
// bits (out_bits) and as fp32 (out_f32), either may be null; *n_out = its element count, 0 if the
// file has no such tensor.  cap = capacity of the buffers in elements.
int fst_file_read_tensor(const char* path, uint32_t tid, int layer, int sub, uint16_t* out_bits, float* out_f32,
                         int64_t cap, int64_t* n_out, int* qtype_out) {
  return guard([&] {
    const std::vector<fstfile::Entry> dir = fstfile::read_directory(path);
    const fstfile::Entry* en = fstfile::find(dir, tid, layer, sub);
    *n_out = 0;
    if (!en) return;
    if (qtype_out) *qtype_out = en->qtype;
    const int64_t n = (int64_t)en->n_elements();
    if (n > cap) throw std::runtime_error("buffer too small for the tensor");
    if (out_bits) {
      const std::vector<uint16_t> v = fstfile::load_bf16(path, *en);
      std::memcpy(out_bits, v.data(), v.size() * 2);
    }
    if (out_f32) {
      const std::vector<float> v = fstfile::load_f32(path, *en);
      std::memcpy(out_f32, v.data(), v.size() * 4);
    }
    *n_out = n;
  });
}
int fst_engine_preload(FSTEngine* e) { return guard([&] { e->preload_all_layers(); }); }
int fst_engine_process_mla(FSTEngine* e, int lid, uint16_t* h, int M) { return guard([&] { e->process_mla(lid, h, M); }); }
int fst_engine_process_mla_batch(FSTEngine* e, int lid, uint16_t* h, const int* seqs, const int* pos0, const int* q_lens,
                                 int B, int causal) {
  return guard([&] { e->process_mla_batch(lid, h, seqs, pos0, q_lens, B, causal != 0); });
}
int fst_engine_reset_session(FSTEngine* e) { return guard([&] { e->reset_session(); }); }
int fst_engine_seq_pos(FSTEngine* e) { return e->seq_pos(); }
void fst_engine_advance(FSTEngine* e, int n) { e->advance(n); }
void fst_engine_set_prefill(FSTEngine* e, int p) { e->set_prefill(p != 0); }
int fst_engine_rollback(FSTEngine* e, int keep) { return guard([&] { e->rollback(keep); }); }
int fst_engine_set_window(FSTEngine* e, int window) { return guard([&] { e->set_window(window); }); }
int fst_engine_new_sequence(FSTEngine* e) {
  int s = -1;
  guard([&] { s = e->new_sequence(); });
  return s;
}
int fst_engine_current_sequence(FSTEngine* e) { return e->current_sequence(); }
// Fills cos / ratio / maxerr for up to cap probes; returns the number of probes or -1.
int fst_engine_randmat_test(FSTEngine* e, double* cosine, double* ratio, double* max_err, int cap) {
  int n = -1;
  guard([&] {
    auto r = e->randmat_test();
    n = 0;
    for (size_t i = 0; i < r.size() && (int)i < cap; ++i, ++n) {
      cosine[i] = r[i].cosine;
      ratio[i] = r[i].norm_ratio;
      max_err[i] = r[i].max_abs_err;
    }
  });
  return n;
}
FstMlaCtx* fst_engine_ctx(FSTEngine* e) { return e->ctx(); }
void fst_engine_set_draft(FSTEngine* e, int window_size) {
  e->config_.draft = true;
  e->config_.window_size = window_size;
}
int fst_engine_process_draft_mla(FSTEngine* e, int lid, uint16_t* h, int M, const uint16_t* main_x) {
  return guard([&] { e->process_draft_mla(lid, h, M, main_x); });
}
void fst_engine_enable_compressor(FSTEngine* e, int on) { e->enable_compressor(on != 0); }
int fst_engine_snapshot_before_verify(FSTEngine* e) { return guard([&] { e->snapshot_before_verify(); }); }
int fst_engine_layer_cmp_ratio(FSTEngine* e, int lid) { return e->shared_.at(lid).cmp_ratio; }
int fst_engine_join_split_group(FSTEngine* e, const uint8_t* id, int rank, int world) {
  return guard([&] { e->join_split_group(id, rank, world); });
}
void fst_engine_set_kv_slice(FSTEngine* e, int slice_begin) { e->set_kv_slice(slice_begin); }
void fst_engine_set_seq_pos(FSTEngine* e, int pos) { e->set_seq_pos(pos); }
int fst_engine_process_mla_split(FSTEngine* e, int lid, uint16_t* h, int M, int owns_new_rows) {
  return guard([&] { e->process_mla_split(lid, h, M, owns_new_rows != 0); });
}
}
