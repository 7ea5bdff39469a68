// Context, paged-cache bookkeeping, split-KV planning and the C ABI of the MLA path.
// Host-side logic only; the kernels live in kernels_simt.cu, gemm_tc.cu and attn_stream.cu.
#include <dlfcn.h>

#include <algorithm>
#include <cmath>
#include <cstdarg>
#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <string>
#include <vector>

#include "../../include/fst_cuda_mla.h"
#include "kernels.cuh"

using namespace fst;

namespace {

thread_local std::string g_err;

}  // namespace

namespace fst {
PerDeviceOnce& kernel_attr_registry() {
  static PerDeviceOnce r;
  return r;
}
void set_last_error(const char* msg) { g_err = msg ? msg : ""; }
}  // namespace fst

namespace {

int fail(int code, const char* fmt, ...) {
  char buf[512];
  va_list ap;
  va_start(ap, fmt);
  vsnprintf(buf, sizeof(buf), fmt, ap);
  va_end(ap);
  g_err = buf;
  return code;
}

#define CU(call)                                                                           \
  do {                                                                                     \
    cudaError_t e_ = (call);                                                               \
    if (e_ != cudaSuccess)                                                                 \
      return fail(FST_MLA_ERR_CUDA, "%s failed: %s (%s:%d)", #call, cudaGetErrorString(e_), \
                  __FILE__, __LINE__);                                                     \
  } while (0)

struct Dims {
  int H, hidden, q_lora, kv_lora, nope, rope, v_head, row, d_qk, d_v, q_head, low, cmp_n;
  bool v4;
};

struct LayerW {
  bf16 *w_cmp = nullptr, *wq_b = nullptr, *wkv_b = nullptr, *wo_a = nullptr, *wo_b = nullptr;
  bf16 *q_norm = nullptr, *kv_norm = nullptr;
  bf16* attn_norm = nullptr;  // [hidden] or null: the norm in front of the layer
  float* sinks = nullptr;
  bool set = false;
  bool draft_form = false;  // the draft model's layer: no per-head q norm, q / output tail rotation on head 0 only
  // V4 KV compressor (reference LayerWeightsC cmp_*, include/fst_engine.h:172-180): 0 = none
  int cmp_ratio = 0;
  bf16* w_cmp_proj = nullptr;   // [2 * width, hidden]: wkv rows, then wgate rows
  float* cmp_ape = nullptr;     // [ratio, width]
  bf16* cmp_norm = nullptr;     // [kv_lora]
  float* cmp_state = nullptr;   // [max_seqs][2][rows, width] window state per sequence (values, scores)
  float* cmp_snap = nullptr;    // the same, saved by fst_cuda_mla_seq_snapshot
  std::vector<int32_t> cmp_pos, cmp_pos_snap;  // per sequence: rows [0, cmp_pos) have gone through the compressor
};

// Layers fall into classes by their compress ratio (0: no compressor, 4, 128): the split-KV
// schedule of a plan differs between classes, because compressed rows are further columns.
constexpr int N_CLASSES = 3;
inline int class_of_ratio(int ratio) { return ratio == 0 ? 0 : ratio == 4 ? 1 : 2; }
constexpr int CLASS_RATIO[N_CLASSES] = {0, 4, 128};

struct Sched {
  bool built = false;
  int32_t *d_cta_seg = nullptr, *d_tok_part = nullptr;
  AttnSeg* d_segs = nullptr;
  int n_segs = 0, n_parts = 0, n_ctas = 0;
  long long kv_rows = 0;
  int max_tok_parts = 0, min_tok_parts = 0, n_single_part = 0;
  bool by_blocks = false;  // cut_block_schedule made it: the lanes of a group read the same pages side by side
  // what the compressor kernel of this class reads (classes 1, 2)
  CompressTok* d_ctoks = nullptr;
  CompressStep* d_csteps = nullptr;
  float* d_lut_cmp = nullptr;
  int n_csteps = 0;
};

constexpr int ATTN_TILE = 128;      // split boundaries are multiples of this many cached rows
constexpr int MAX_EVENT_SETS = 256;

struct EventSet {
  cudaEvent_t ev[FST_MLA_K_COUNT + 1];
  bool used[FST_MLA_K_COUNT + 1];
};

}  // namespace

struct FstMlaCtx {
  FstMlaConfig cfg;
  Dims d;
  int n_sm = 0;
  cudaStream_t stream = nullptr;
  std::vector<LayerW> layers;
  std::vector<bf16*> pools;  // per layer [n_pages * page_tokens, row]

  // paged-cache bookkeeping (host)
  std::vector<int32_t> free_pages, free_seqs;
  std::vector<std::vector<int32_t>> tables;
  std::vector<int32_t> lens;
  std::vector<char> live;

  // workspaces
  bf16* d_an = nullptr;  // [T, hidden] rows after attn_norm (layers that carry the weight)
  bf16 *d_h = nullptr, *d_cmp = nullptr, *d_qc = nullptr, *d_kvnew = nullptr, *d_qfull = nullptr;
  bf16 *d_qeff = nullptr, *d_olat = nullptr, *d_low = nullptr, *d_out = nullptr;
  float *d_part_m = nullptr, *d_part_l = nullptr, *d_part_o = nullptr;
  int max_parts = 0;
  bool fused_merge = true;       // the attention kernel finishes single-partial tokens itself
  bool block_schedule = true;    // calls with G >= 4 new tokens per sequence: thread blocks in groups of G lanes
  Sched sched[N_CLASSES];        // the current plan's schedule per layer class
  int info_class = 0;            // class of the layer that ran last (plan_info reports its schedule)
  bool has_cmp = false;          // some layer has a KV compressor
  int cmp_min_ratio = 0;         // the smallest compress ratio in use: sizes the compressed-row pages
  std::vector<std::vector<int32_t>> comp_tables;  // per sequence: pages of its compressed rows (all layers)
  std::vector<int32_t> snap_len;                  // per sequence: length at its snapshot, or -1
  bf16* d_cproj = nullptr;       // [T, 2 * width] compressor projections of a call
  uint16_t* h_pinned = nullptr;  // [max_tokens, hidden] staging for the host-buffer entry point
  int* d_status = nullptr;
  const bf16* out_src = nullptr;  // where the last layer call left its output rows
  bool out_zero_copy = true;
  int* h_status = nullptr;  // page-locked copy of the status word, fetched on the stream before a sync
  int* h_status_dev = nullptr;   // the device's address of h_status (mapped), or null
  bool status_by_kernel = false; // the last kernel enqueued was an O-proj b that stores the status word to h_status itself

  // RoPE kind of every layer: 0 plain (theta = cfg.rope_theta), 1 YaRN (reference
  // build_rope_lut picks per layer, src/fst_engine.cpp:1979-1982)
  std::vector<int8_t> layer_yarn;
  // plan (device)
  float* d_lut_k[2] = {nullptr, nullptr};  // [T, rope] (cos, sin) per RoPE kind that some layer uses
  long long* d_dst = nullptr;
  int32_t* d_tables = nullptr;
  int tables_cap = 0, segs_cap = 0;
  // the plan arrays above are slices of one device blob, filled through one pinned host blob
  // with a single copy per plan
  unsigned char *d_plan = nullptr, *h_plan = nullptr;
  size_t plan_cap = 0;
  cudaEvent_t plan_ev = nullptr;
  // RoPE table rows by position, direct-mapped: one step of a model asks for the same positions
  // in every layer, and a decode step for the positions right after the previous step's
  std::vector<float> lut_rows[2];  // per RoPE kind
  std::vector<int32_t> lut_tag[2];
  // plan (host): the per-token arrays live here between the two phases of a plan
  std::vector<float> pl_lut[2];
  std::vector<long long> pl_dst;
  std::vector<int32_t> pl_tok_table, pl_tables, pl_kvlen, pl_kvlo, pl_tok_ctable, pl_tok_step;
  std::vector<FstMlaSeqStep> pl_steps;
  int pl_causal = 0;
  size_t pl_off_b = 0;          // where the second part of the blob starts
  bool front_uploaded = false;  // the first part (RoPE rows, append addresses) went ahead on its own
  cudaStream_t copy_stream = nullptr;  // carries the second part while the front kernels run
  cudaEvent_t plan_ev_b = nullptr, fwd_ev = nullptr;
  std::vector<FstMlaSeqStep> last_steps;  // what the valid plan was built from (every layer of a
  int last_causal = 0;                    // model step asks for the same plan again)
  bool plan_reuse = true;
  int32_t window = 0;  // sliding window applied by fst_cuda_mla_forward (0: none)
  int64_t plans_built = 0, plans_reused = 0;
  bool planned = false;
  int T = 0;

  // split-KV across GPUs: the exchange of the per-GPU partials
  void* nccl_comm = nullptr;         // ncclComm_t
  FstMlaGatherFn gather_fn = nullptr;  // host-supplied transport instead
  void* gather_user = nullptr;
  int comm_rank = 0, comm_world = 0;
  float *d_xpart = nullptr, *d_xgath = nullptr;  // [T*H, 2 + d_v] and [world][T*H, 2 + d_v]

  int64_t launches = 0;
  int64_t launches_tensor = 0, launches_simt = 0;  // GEMM / attention launches by kernel family
  bool profiling = false;
  bool compress_done = false;  // fst_cuda_mla_forward has launched the compress GEMM of this call already
  std::vector<EventSet> ev_pool;
  int ev_used = 0;
  float k_ms[FST_MLA_K_COUNT] = {0};
  int32_t k_n[FST_MLA_K_COUNT] = {0};
  EventSet* cur = nullptr;
};

namespace {

void comm_release(FstMlaCtx* c);  // (defined with the exchange code below)

Dims dims_of(const FstMlaConfig& c) {
  Dims d;
  d.v4 = c.preset == FST_MLA_PRESET_FASTAR_V4;
  d.H = c.n_heads;
  d.hidden = c.hidden;
  d.q_lora = c.q_lora;
  d.kv_lora = c.kv_lora;
  d.rope = c.qk_rope;
  if (!d.v4) {
    d.nope = c.qk_nope;
    d.v_head = c.v_head;
    d.row = c.kv_lora + c.qk_rope;
    d.d_qk = d.row;
    d.d_v = c.kv_lora;
    d.q_head = c.qk_nope + c.qk_rope;
    d.low = c.n_heads * c.v_head;
  } else {
    d.nope = c.kv_lora - c.qk_rope;
    d.v_head = 0;
    d.row = c.kv_lora;
    d.d_qk = c.kv_lora;
    d.d_v = c.kv_lora;
    d.q_head = c.kv_lora;
    d.low = c.o_groups * c.o_lora;
  }
  d.cmp_n = d.q_lora + d.row;
  return d;
}

// RoPE table of one position, the recurrence of build_rope_lut (reference
// src/fst_engine.cpp:1970-2023): theta_0 = pos, theta_{j+1} = theta_j * base^(-2/rope_dim) in
// fp32; YaRN layers mix theta/16 and theta through the correction ramp (1995-2022).  The
// table stays fp32 (the reference rounds it to bf16, 1988-1989).
void rope_lut_row(float* lut, int pos, int rope_dim, float theta, bool yarn) {
  const float freq_base = yarn ? 160000.0f : theta;
  const float theta_scale = std::pow(freq_base, -2.0f / (float)rope_dim);
  float th = (float)pos;
  float corr0 = 0, corr1 = 0;
  if (yarn) {
    auto corr_dim = [&](float beta) {
      return (float)rope_dim * std::log(65536.0f / (beta * 2.0f * (float)M_PI)) / (2.0f * std::log(freq_base));
    };
    corr0 = std::max(0.0f, std::floor(corr_dim(32.0f)));
    corr1 = std::min((float)(rope_dim - 1), std::ceil(corr_dim(1.0f)));
  }
  for (int dd = 0; dd < rope_dim; dd += 2) {
    float ang = th;
    if (yarn) {
      const float y = ((float)(dd / 2) - corr0) / std::max(0.001f, corr1 - corr0);
      const float mix = 1.0f - std::min(1.0f, std::max(0.0f, y));
      ang = (th / 16.0f) * (1.0f - mix) + th * mix;
    }
    sincosf(ang, &lut[dd + 1], &lut[dd]);  // bit-identical to sinf / cosf (checked over 25.6 M angles), one call
    th *= theta_scale;
  }
}

constexpr int LUT_CACHE_ROWS = 4096;  // power of two

// the RoPE row of one position, computed on its first use and kept until another position maps to
// the same slot
const float* lut_row_cached(FstMlaCtx* c, int kind, int pos) {
  const int rope = c->d.rope;
  if (c->lut_tag[kind].empty()) {
    c->lut_tag[kind].assign(LUT_CACHE_ROWS, -1);
    c->lut_rows[kind].resize((size_t)LUT_CACHE_ROWS * rope);
  }
  const int slot = pos & (LUT_CACHE_ROWS - 1);
  float* row = &c->lut_rows[kind][(size_t)slot * rope];
  if (c->lut_tag[kind][slot] != pos) {
    rope_lut_row(row, pos, rope, c->cfg.rope_theta, kind != 0);
    c->lut_tag[kind][slot] = pos;
  }
  return row;
}

// which RoPE kinds the layers of this context use
void rope_kinds(const FstMlaCtx* c, bool need[2]) {
  need[0] = need[1] = false;
  for (int8_t k : c->layer_yarn) need[k ? 1 : 0] = true;
}
const float* lut_of(const FstMlaCtx* c, int lid) { return c->d_lut_k[c->layer_yarn[lid] ? 1 : 0]; }
// heads whose output tail gets the inverse rotation (reference 3716; the draft layer: head 0, 5077-5093)
int inv_rope_heads(const FstMlaCtx* c, int lid) { return !c->d.v4 ? 0 : c->layers[lid].draft_form ? 1 : c->d.H; }
int class_of(const FstMlaCtx* c, int lid) { return class_of_ratio(c->layers[lid].cmp_ratio); }
Sched& sched_of(FstMlaCtx* c, int lid) { return c->sched[class_of(c, lid)]; }
int cmp_width(const FstMlaCtx* c, int ratio) { return ratio == 4 ? 2 * c->d.kv_lora : c->d.kv_lora; }
int cmp_rows(int ratio) { return ratio == 4 ? 8 : ratio; }
size_t cmp_slot_floats(const FstMlaCtx* c, int ratio) { return (size_t)2 * cmp_rows(ratio) * cmp_width(c, ratio); }

bool seq_ok(const FstMlaCtx* c, int32_t s) { return s >= 0 && s < c->cfg.max_seqs && c->live[s]; }

int reserve_pages(FstMlaCtx* c, int32_t seq, int32_t n_tokens) {
  const size_t need = ((size_t)n_tokens + c->cfg.page_tokens - 1) / c->cfg.page_tokens;
  auto& t = c->tables[seq];
  if (need > t.size() && need - t.size() > c->free_pages.size())
    return fail(FST_MLA_ERR_PAGES, "page pool exhausted: sequence %d needs %zu more pages, %zu free", seq,
                need - t.size(), c->free_pages.size());
  // layers with a KV compressor keep one compressed row per `ratio` rows, in pages of their own
  auto& ct = c->comp_tables[seq];
  const size_t need_c = c->has_cmp ? ((size_t)(n_tokens / c->cmp_min_ratio) + c->cfg.page_tokens - 1) / c->cfg.page_tokens : 0;
  const size_t more = (need > t.size() ? need - t.size() : 0) + (need_c > ct.size() ? need_c - ct.size() : 0);
  if (more > c->free_pages.size())
    return fail(FST_MLA_ERR_PAGES, "page pool exhausted: sequence %d needs %zu more pages, %zu free", seq, more,
                c->free_pages.size());
  while (t.size() < need) {
    t.push_back(c->free_pages.back());
    c->free_pages.pop_back();
  }
  while (ct.size() < need_c) {
    ct.push_back(c->free_pages.back());
    c->free_pages.pop_back();
  }
  c->lens[seq] = std::max(c->lens[seq], n_tokens);
  return FST_MLA_OK;
}

long long row_offset(const FstMlaCtx* c, int32_t seq, int32_t pos) {
  const int pt = c->cfg.page_tokens;
  return ((long long)c->tables[seq][pos / pt] * pt + pos % pt) * c->d.row;
}

template <class T>
int dev_alloc(T** p, size_t n) {
  CU(cudaMalloc((void**)p, std::max<size_t>(n, 1) * sizeof(T)));
  return FST_MLA_OK;
}

void prof_mark(FstMlaCtx* c, int k) {
  if (!c->cur) return;
  cudaEventRecord(c->cur->ev[k], c->stream);
  c->cur->used[k] = true;
}

int prof_flush(FstMlaCtx* c) {
  if (c->ev_used == 0) return FST_MLA_OK;
  CU(cudaStreamSynchronize(c->stream));
  for (int i = 0; i < c->ev_used; ++i) {
    EventSet& es = c->ev_pool[i];
    // a kernel's time runs from its own mark to the next mark that was recorded
    for (int k = 0; k < FST_MLA_K_COUNT; ++k) {
      if (!es.used[k]) continue;
      int nx = k + 1;
      while (nx <= FST_MLA_K_COUNT && !es.used[nx]) ++nx;
      if (nx > FST_MLA_K_COUNT) continue;
      float ms = 0;
      if (cudaEventElapsedTime(&ms, es.ev[k], es.ev[nx]) == cudaSuccess) {
        c->k_ms[k] += ms;
        c->k_n[k] += 1;
      }
    }
    memset(es.used, 0, sizeof(es.used));
  }
  c->ev_used = 0;
  return FST_MLA_OK;
}

int prof_begin(FstMlaCtx* c) {
  c->cur = nullptr;
  if (!c->profiling) return FST_MLA_OK;
  if (c->ev_used == MAX_EVENT_SETS) {
    int rc = prof_flush(c);
    if (rc) return rc;
  }
  if ((int)c->ev_pool.size() <= c->ev_used) {
    EventSet es;
    memset(es.used, 0, sizeof(es.used));
    for (auto& e : es.ev) CU(cudaEventCreate(&e));
    c->ev_pool.push_back(es);
  }
  c->cur = &c->ev_pool[c->ev_used++];
  return FST_MLA_OK;
}

bool use_tc_gemm(const FstMlaCtx* c, const GemmArgs& g) {
  if (c->cfg.gemm_impl == FST_MLA_IMPL_SIMT) return false;
  return gemm_tc_supported(g);
}

int run_gemm(FstMlaCtx* c, const GemmArgs& g) {
  c->status_by_kernel = false;
  if (c->cfg.gemm_impl == FST_MLA_IMPL_TENSOR && !gemm_tc_supported(g))
    return fail(FST_MLA_ERR_ARG, "GEMM %dx%dx%d (b_kn=%d) has no tcgen05 path", g.M, g.N, g.K, g.b_kn);
  if (use_tc_gemm(c, g)) {
    cudaError_t e = launch_gemm_tc(g, c->d_status, c->stream);
    if (e != cudaSuccess) return fail(FST_MLA_ERR_CUDA, "tcgen05 GEMM launch: %s", cudaGetErrorString(e));
    c->launches_tensor += 1;
  } else {
    launch_gemm_simt(g, c->stream);
    c->launches_simt += 1;
  }
  c->launches += 1;
  return FST_MLA_OK;
}

GemmArgs plain_gemm(const bf16* A, const bf16* B, bf16* C, int M, int N, int K) {
  GemmArgs g;
  g.A = A; g.B = B; g.C = C;
  g.M = M; g.N = N; g.K = K;
  g.lda = K; g.ldb = K; g.ldc = N;
  g.batch = 1; g.a_bs = g.b_bs = g.c_bs = 0;
  g.b_kn = 0;
  return g;
}

AttnArgs attn_args(FstMlaCtx* c, int lid, const bf16* q_eff, bool may_fuse = false) {
  AttnArgs a;
  a.q_eff = q_eff;
  a.pool = c->pools[lid];
  a.tables = c->d_tables;
  const Sched& S = sched_of(c, lid);
  a.segs = S.d_segs;
  a.cta_seg = S.d_cta_seg;
  a.part_m = c->d_part_m;
  a.part_l = c->d_part_l;
  a.part_o = c->d_part_o;
  a.d_status = c->d_status;
  a.n_segs = S.n_segs;
  a.n_ctas = S.n_ctas;
  a.H = c->d.H;
  a.d_qk = c->d.d_qk;
  a.d_v = c->d.d_v;
  a.row = c->d.row;
  a.page_tokens = c->cfg.page_tokens;
  a.pool_rows = (long long)c->cfg.n_pages * c->cfg.page_tokens;
  a.q_rows = (long long)c->T * c->d.H;
  a.scale = c->cfg.softmax_scale;
  a.tiles_shared = S.by_blocks;
  if (may_fuse && c->fused_merge && S.n_single_part > 0) {
    a.direct_single = true;
    a.tok_part = S.d_tok_part;
    a.o_lat = c->d_olat;
    a.sinks = c->d.v4 ? c->layers[lid].sinks : nullptr;
    a.lut = lut_of(c, lid);
    a.rope = c->d.rope;
    a.inv_rope = inv_rope_heads(c, lid);
  }
  return a;
}

// *direct (if given; mode-0 callers): the attention kernel has written the o_lat rows of every
// token that has exactly one partial; the merge that follows skips them.
int run_attention(FstMlaCtx* c, int lid, const bf16* q_eff, bool* direct = nullptr) {
  if (direct) *direct = false;
  c->status_by_kernel = false;
  c->info_class = class_of(c, lid);
  if (sched_of(c, lid).n_segs == 0) return FST_MLA_OK;
  AttnArgs a = attn_args(c, lid, q_eff, direct != nullptr);
  const bool tc_ok = attn_stream_supported(a);
  if (!(c->cfg.attn_impl != FST_MLA_IMPL_SIMT && tc_ok)) a.direct_single = false;
  if (direct) *direct = a.direct_single;
  if (c->cfg.attn_impl == FST_MLA_IMPL_TENSOR && !tc_ok)
    return fail(FST_MLA_ERR_ARG, "this shape has no tcgen05 attention path");
  if (c->cfg.attn_impl != FST_MLA_IMPL_SIMT && tc_ok) {
    cudaError_t e = launch_attn_stream(a, c->stream);
    if (e != cudaSuccess) return fail(FST_MLA_ERR_CUDA, "tcgen05 attention launch: %s", cudaGetErrorString(e));
    c->launches_tensor += 1;
  } else {
    launch_attn_simt(a, c->stream);
    c->launches_simt += 1;
  }
  c->launches += 1;
  return FST_MLA_OK;
}

// Stages before the attention: projections, norms, RoPE, cache append, absorbed query.
int run_front(FstMlaCtx* c, int lid, const bf16* h_in) {
  const Dims& d = c->d;
  const LayerW& w = c->layers[lid];
  const int T = c->T;
  int rc;
  prof_mark(c, FST_MLA_K_COMPRESS);
  if (w.attn_norm && !c->compress_done) {
    // attn_norm of process_layer (reference 2687-2688) in front of the compressions
    launch_rmsnorm_rows(h_in, w.attn_norm, c->d_an, T, d.hidden, c->cfg.rms_eps, c->stream);
    c->launches += 1;
    h_in = c->d_an;
  }
  if (!c->compress_done && (rc = run_gemm(c, plain_gemm(h_in, w.w_cmp, c->d_cmp, T, d.cmp_n, d.hidden)))) return rc;
  c->compress_done = false;
  if (w.cmp_ratio) {
    // KV compressor (reference 3545-3568): the rows' two projections as one GEMM, then the state
    // machine of every sequence, its rows in order; compressed rows land in their pages before the
    // attention reads them
    const Sched& S = sched_of(c, lid);
    const int width = cmp_width(c, w.cmp_ratio);
    for (const FstMlaSeqStep& st : c->pl_steps) {
      if (st.q_len == 0) continue;
      if (!st.append) return fail(FST_MLA_ERR_STATE, "layer %d has a KV compressor: its sequences must own their new rows", lid);
      if (w.cmp_pos[st.seq] != st.pos0)
        return fail(FST_MLA_ERR_STATE,
                    "layer %d: the compressor of sequence %d has seen rows [0, %d), the call starts at row %d "
                    "(rows must arrive in order; fst_cuda_mla_seq_snapshot / _truncate undo a block)",
                    lid, st.seq, w.cmp_pos[st.seq], st.pos0);
    }
    if ((rc = run_gemm(c, plain_gemm(h_in, w.w_cmp_proj, c->d_cproj, T, 2 * width, d.hidden)))) return rc;
    CompressArgs ca;
    ca.proj = c->d_cproj; ca.ape = w.cmp_ape; ca.norm = w.cmp_norm; ca.lut = S.d_lut_cmp; ca.toks = S.d_ctoks;
    ca.steps = S.d_csteps; ca.state = w.cmp_state; ca.pool = c->pools[lid]; ca.n_steps = S.n_csteps;
    ca.ratio = w.cmp_ratio; ca.width = width; ca.kv_lora = d.kv_lora; ca.rope = d.rope;
    launch_compress(ca, c->stream);
    c->launches += 1;
    for (const FstMlaSeqStep& st : c->pl_steps) c->layers[lid].cmp_pos[st.seq] = st.pos0 + st.q_len;
  }
  prof_mark(c, FST_MLA_K_NORM_APPEND);
  NormAppendArgs na;
  na.cmp = c->d_cmp; na.q_norm = w.q_norm; na.kv_norm = w.kv_norm; na.lut = lut_of(c, lid);
  na.dst_row = c->d_dst; na.qc = c->d_qc; na.kv_new = c->d_kvnew; na.pool = c->pools[lid];
  na.T = T; na.q_lora = d.q_lora; na.kv_lora = d.kv_lora; na.row = d.row; na.rope = d.rope;
  na.eps = c->cfg.rms_eps;
  launch_norm_append(na, c->stream);
  c->launches += 1;
  prof_mark(c, FST_MLA_K_Q_EXPAND);
  if ((rc = run_gemm(c, plain_gemm(c->d_qc, w.wq_b, c->d_qfull, T, d.H * d.q_head, d.q_lora)))) return rc;
  prof_mark(c, FST_MLA_K_Q_ABSORB);
  QPrepArgs qp;
  qp.q_full = c->d_qfull; qp.lut = lut_of(c, lid); qp.q_eff = c->d_qeff;
  qp.T = T; qp.H = d.H; qp.q_head = d.q_head; qp.nope = d.nope; qp.rope = d.rope; qp.d_qk = d.d_qk;
  qp.v4 = d.v4; qp.eps = c->cfg.rms_eps;
  if (w.draft_form) {
    qp.head_norm = 0;
    qp.rope_heads = 1;
  }
  if (d.v4) {
    launch_q_prep(qp, c->stream);
    c->launches += 1;
  } else {
    // q_lat[h] = q_nope[h] (128) * W_UK[h] ([128, 512], a [K, N] operand), one batch member per head
    GemmArgs g;
    g.A = c->d_qfull; g.B = w.wkv_b; g.C = c->d_qeff;
    g.M = T; g.N = d.kv_lora; g.K = d.nope;
    g.lda = d.H * d.q_head; g.ldb = d.kv_lora; g.ldc = d.H * d.d_qk;
    g.batch = d.H; g.a_bs = d.q_head; g.b_bs = (long long)(d.nope + d.v_head) * d.kv_lora; g.c_bs = d.d_qk;
    g.b_kn = 1;
    const bool even = d.q_head % 2 == 0 && d.nope % 2 == 0 && d.d_qk % 2 == 0 && d.rope % 2 == 0;
    if (use_tc_gemm(c, g) && even) {
      // the q_pe RoPE rides in the same kernel: it reads the same input and fills the other
      // columns of q_eff, and a kernel boundary costs more than the rotation itself
      g.rope_src = c->d_qfull; g.rope_lut = lut_of(c, lid); g.rope_dst = c->d_qeff;
      g.rope_T = T; g.rope_H = d.H; g.rope_q_head = d.q_head; g.rope_nope = d.nope; g.rope_dims = d.rope;
      g.rope_d_qk = d.d_qk;
    } else {
      launch_q_prep(qp, c->stream);
      c->launches += 1;
    }
    if ((rc = run_gemm(c, g))) return rc;
  }
  return FST_MLA_OK;
}

// Output projections a and b.
int run_back(FstMlaCtx* c, int lid, bf16* h_out) {
  const Dims& d = c->d;
  const LayerW& w = c->layers[lid];
  const int T = c->T;
  int rc;
  prof_mark(c, FST_MLA_K_OPROJ_A);
  GemmArgs g;
  g.A = c->d_olat; g.C = c->d_low; g.M = T; g.b_kn = 0;
  g.lda = d.H * d.d_v; g.ldc = d.low;
  if (d.v4) {
    // 8 groups: low[:, g*o_lora:] = heads[:, g*gk:(g+1)*gk] * wo_a[g]^T (reference 3736-3839)
    const int gk = d.H * d.d_v / c->cfg.o_groups;
    g.B = w.wo_a; g.N = c->cfg.o_lora; g.K = gk; g.ldb = gk;
    g.batch = c->cfg.o_groups; g.a_bs = gk; g.b_bs = (long long)c->cfg.o_lora * gk; g.c_bs = c->cfg.o_lora;
  } else {
    // per-head W_UV: low[:, h*v_head:] = o_lat[:, h, :] * W_UV[h]^T
    g.B = w.wkv_b + (long long)d.nope * d.kv_lora; g.N = d.v_head; g.K = d.d_v; g.ldb = d.kv_lora;
    g.batch = d.H; g.a_bs = d.d_v; g.b_bs = (long long)(d.nope + d.v_head) * d.kv_lora; g.c_bs = d.v_head;
  }
  if ((rc = run_gemm(c, g))) return rc;
  prof_mark(c, FST_MLA_K_OPROJ_B);
  GemmArgs gb = plain_gemm(c->d_low, w.wo_b, h_out, T, d.hidden, d.low);
  const bool by_kernel = c->h_status_dev && use_tc_gemm(c, gb);
  if (by_kernel) {
    gb.status_dev = c->d_status;
    gb.status_host = c->h_status_dev;
  }
  if ((rc = run_gemm(c, gb))) return rc;
  c->status_by_kernel = by_kernel;  // (until anything else is launched: run_gemm clears it)
  prof_mark(c, FST_MLA_K_COUNT);
  return FST_MLA_OK;
}

// skip_single: the attention kernel finished the single-partial tokens; when every token with a
// context is one, nothing is left to merge (tokens without any context still get their zero /
// sink-only rows from the merge kernel).
int run_merge_local(FstMlaCtx* c, int lid, int mode, float* rank_partial, bool skip_single = false) {
  const Dims& d = c->d;
  const Sched& S = sched_of(c, lid);
  if (skip_single && S.min_tok_parts == 1 && S.max_tok_parts == 1) return FST_MLA_OK;
  MergeArgs m;
  m.skip_single = skip_single ? 1 : 0;
  m.part_m = c->d_part_m; m.part_l = c->d_part_l; m.part_o = c->d_part_o; m.tok_part = S.d_tok_part;
  m.sinks = (d.v4 && mode == 0) ? c->layers[lid].sinks : nullptr;
  m.lut = lut_of(c, lid); m.o_lat = c->d_olat; m.rank_partial = rank_partial;
  m.T = c->T; m.H = d.H; m.d_v = d.d_v; m.rope = d.rope; m.inv_rope = inv_rope_heads(c, lid); m.mode = mode;
  m.threads = S.n_parts <= 6 * c->T ? 128 : 256;
  m.wide = (long long)c->T * d.H < 2ll * c->n_sm ? 1 : 0;  // too few rows to fill the SMs with a block each
  launch_merge(m, c->stream);
  c->launches += 1;
  return FST_MLA_OK;
}

int check_run(FstMlaCtx* c, int lid) {
  if (!c) return fail(FST_MLA_ERR_ARG, "null context");
  if (lid < 0 || lid >= c->cfg.n_layers) return fail(FST_MLA_ERR_ARG, "layer %d out of range", lid);
  if (!c->layers[lid].set) return fail(FST_MLA_ERR_STATE, "layer %d has no weights", lid);
  if (!c->planned) return fail(FST_MLA_ERR_STATE, "no plan: call fst_cuda_mla_plan first");
  return FST_MLA_OK;
}

}  // namespace

extern "C" {

const char* fst_cuda_mla_last_error(void) { return g_err.c_str(); }

int fst_cuda_mla_create(const FstMlaConfig* cfg, FstMlaCtx** out) {
  if (!cfg || !out) return fail(FST_MLA_ERR_ARG, "null argument");
  *out = nullptr;
  FstMlaConfig c = *cfg;
  if (c.preset != FST_MLA_PRESET_BASELINE && c.preset != FST_MLA_PRESET_FASTAR_V4)
    return fail(FST_MLA_ERR_ARG, "unknown preset %d", c.preset);
  if (c.hidden <= 0 || c.n_heads <= 0 || c.q_lora <= 0 || c.kv_lora <= 0 || c.qk_rope <= 0 ||
      c.qk_rope % 2 || c.n_layers <= 0 || c.page_tokens <= 0 || c.n_pages <= 0 || c.max_seqs <= 0 ||
      c.max_tokens <= 0)
    return fail(FST_MLA_ERR_ARG, "non-positive dimension in FstMlaConfig");
  if (c.preset == FST_MLA_PRESET_BASELINE && (c.qk_nope <= 0 || c.v_head <= 0))
    return fail(FST_MLA_ERR_ARG, "BASELINE preset needs qk_nope and v_head");
  if (c.preset == FST_MLA_PRESET_FASTAR_V4 &&
      (c.o_groups <= 0 || c.o_lora <= 0 || (c.n_heads * c.kv_lora) % c.o_groups || c.qk_rope >= c.kv_lora))
    return fail(FST_MLA_ERR_ARG, "V4 preset needs o_groups dividing n_heads*kv_lora and o_lora");
  Dims d = dims_of(c);
  if (d.row % 8 || d.d_qk % 8 || d.d_v % 64 || d.d_v > 512 || d.q_head > 1024 || d.row > 1024)
    return fail(FST_MLA_ERR_ARG, "row width must be a multiple of 8 and d_v a multiple of 64 (<= 512)");
  if (c.q_lora > 2048 || c.qk_rope > 512 || c.hidden > 8192)
    return fail(FST_MLA_ERR_ARG, "q_lora above 2048, rope dims above 512 or hidden above 8192: beyond the register tiles of the norm kernels");
  if (c.softmax_scale <= 0)
    c.softmax_scale = 1.0f / std::sqrt((float)(d.v4 ? c.kv_lora : c.qk_nope + c.qk_rope));
  if (c.rope_theta <= 0) c.rope_theta = 10000.0f;
  if (c.rms_eps <= 0) c.rms_eps = 1e-6f;

  int n_dev = 0;
  if (cudaGetDeviceCount(&n_dev) != cudaSuccess || n_dev == 0) {
    cudaGetLastError();
    return fail(FST_MLA_ERR_NO_DEVICE, "no CUDA device: this path has no CPU fallback");
  }
  if (c.device < 0 || c.device >= n_dev) return fail(FST_MLA_ERR_ARG, "device %d of %d", c.device, n_dev);
  CU(cudaSetDevice(c.device));
  cudaDeviceProp prop;
  CU(cudaGetDeviceProperties(&prop, c.device));
  if (prop.major != 10)
    return fail(FST_MLA_ERR_NO_DEVICE, "device %d is sm_%d%d; this library is built for sm_100a only",
                c.device, prop.major, prop.minor);

  FstMlaCtx* x = new FstMlaCtx;
  x->cfg = c;
  x->d = d;
  x->n_sm = prop.multiProcessorCount;
  x->layers.resize(c.n_layers);
  x->layer_yarn.assign(c.n_layers, c.rope_yarn ? 1 : 0);
  x->pools.assign(c.n_layers, nullptr);
  for (int i = c.n_pages - 1; i >= 0; --i) x->free_pages.push_back(i);
  for (int i = c.max_seqs - 1; i >= 0; --i) x->free_seqs.push_back(i);
  x->tables.resize(c.max_seqs);
  x->comp_tables.resize(c.max_seqs);
  x->snap_len.assign(c.max_seqs, -1);
  x->lens.assign(c.max_seqs, 0);
  x->live.assign(c.max_seqs, 0);
  *out = x;  // from here on destroy() cleans up after a failure

  const size_t pool_elems = (size_t)c.n_pages * c.page_tokens * d.row;
  const size_t T = c.max_tokens;
  int rc = FST_MLA_OK;
  for (int l = 0; l < c.n_layers && !rc; ++l) {
    rc = dev_alloc(&x->pools[l], pool_elems);
    if (!rc && cudaMemset(x->pools[l], 0, pool_elems * sizeof(bf16)) != cudaSuccess)
      rc = fail(FST_MLA_ERR_CUDA, "cudaMemset(pool) failed");
  }
  // partials: one per thread block plus one per stream of tiles that starts inside a block's run; a
  // token has one stream, two in layers with a KV compressor (V4 form only)
  x->max_parts = x->n_sm + (int)T * (d.v4 ? 2 : 1);
  if (!rc) rc = dev_alloc(&x->d_h, T * d.hidden);
  if (!rc) rc = dev_alloc(&x->d_cmp, T * d.cmp_n);
  if (!rc) rc = dev_alloc(&x->d_an, T * d.hidden);
  if (!rc) rc = dev_alloc(&x->d_qc, T * d.q_lora);
  if (!rc) rc = dev_alloc(&x->d_kvnew, T * d.row);
  if (!rc) rc = dev_alloc(&x->d_qfull, T * d.H * d.q_head);
  if (!rc) rc = dev_alloc(&x->d_qeff, T * d.H * d.d_qk);
  if (!rc) rc = dev_alloc(&x->d_olat, T * d.H * d.d_v);
  if (!rc) rc = dev_alloc(&x->d_low, T * d.low);
  if (!rc) rc = dev_alloc(&x->d_out, T * d.hidden);
  if (!rc && d.v4) rc = dev_alloc(&x->d_cproj, T * 4 * d.kv_lora);
  if (!rc) rc = dev_alloc(&x->d_part_m, (size_t)x->max_parts * d.H);
  if (!rc) rc = dev_alloc(&x->d_part_l, (size_t)x->max_parts * d.H);
  if (!rc) rc = dev_alloc(&x->d_part_o, (size_t)x->max_parts * d.H * d.d_v);
  x->segs_cap = x->max_parts;
  x->tables_cap = c.n_pages + c.max_seqs;
  // first part: two RoPE tables, append addresses, per compressed class the compressor's inputs;
  // second part: per class (token partial ranges, block ranges, segments), then the block tables
  x->plan_cap = 2 * T * d.rope * sizeof(float) + T * sizeof(long long) +
                2 * (T * sizeof(CompressTok) + (size_t)c.max_seqs * sizeof(CompressStep) + T * d.rope * sizeof(float)) +
                N_CLASSES * ((T + 1) * sizeof(int32_t) + ((size_t)x->n_sm + 1) * sizeof(int32_t) +
                             (size_t)x->segs_cap * sizeof(AttnSeg)) +
                (size_t)x->tables_cap * sizeof(int32_t) + 32 * 256;
  if (!rc) rc = dev_alloc(&x->d_plan, x->plan_cap);
  if (!rc && cudaHostAlloc((void**)&x->h_plan, x->plan_cap, cudaHostAllocDefault) != cudaSuccess)
    rc = fail(FST_MLA_ERR_CUDA, "cudaHostAlloc(plan) failed");
  if (!rc && (cudaEventCreateWithFlags(&x->plan_ev, cudaEventDisableTiming) != cudaSuccess ||
              cudaEventCreateWithFlags(&x->plan_ev_b, cudaEventDisableTiming) != cudaSuccess ||
              cudaEventCreateWithFlags(&x->fwd_ev, cudaEventDisableTiming) != cudaSuccess))
    rc = fail(FST_MLA_ERR_CUDA, "cudaEventCreate failed");
  if (!rc && cudaStreamCreateWithFlags(&x->copy_stream, cudaStreamNonBlocking) != cudaSuccess)
    rc = fail(FST_MLA_ERR_CUDA, "cudaStreamCreate failed");
  if (!rc) rc = dev_alloc(&x->d_status, 1);
  if (!rc && cudaMemset(x->d_status, 0, sizeof(int)) != cudaSuccess) rc = fail(FST_MLA_ERR_CUDA, "cudaMemset failed");
  if (!rc && cudaHostAlloc((void**)&x->h_status, sizeof(int), cudaHostAllocMapped) != cudaSuccess)
    rc = fail(FST_MLA_ERR_CUDA, "cudaHostAlloc failed");
  if (!rc) *x->h_status = 0;
  if (!rc && cudaHostGetDevicePointer((void**)&x->h_status_dev, x->h_status, 0) != cudaSuccess) {
    cudaGetLastError();
    x->h_status_dev = nullptr;  // no mapping: the status word is copied behind every call instead
  }
  if (!rc && cudaHostAlloc((void**)&x->h_pinned, T * d.hidden * sizeof(uint16_t), cudaHostAllocDefault) != cudaSuccess)
    rc = fail(FST_MLA_ERR_CUDA, "cudaHostAlloc failed");
  if (rc) {
    std::string keep = g_err;
    fst_cuda_mla_destroy(x);
    *out = nullptr;
    g_err = keep;
    return rc;
  }
  return FST_MLA_OK;
}

void fst_cuda_mla_destroy(FstMlaCtx* c) {
  if (!c) return;
  cudaSetDevice(c->cfg.device);
  cudaDeviceSynchronize();
  comm_release(c);
  for (auto& l : c->layers) {
    cudaFree(l.w_cmp); cudaFree(l.wq_b); cudaFree(l.wkv_b); cudaFree(l.wo_a); cudaFree(l.wo_b);
    cudaFree(l.q_norm); cudaFree(l.kv_norm); cudaFree(l.sinks); cudaFree(l.attn_norm);
    cudaFree(l.w_cmp_proj); cudaFree(l.cmp_ape); cudaFree(l.cmp_norm); cudaFree(l.cmp_state); cudaFree(l.cmp_snap);
  }
  cudaFree(c->d_cproj);
  for (auto p : c->pools) cudaFree(p);
  cudaFree(c->d_an);
  cudaFree(c->d_h); cudaFree(c->d_cmp); cudaFree(c->d_qc); cudaFree(c->d_kvnew); cudaFree(c->d_qfull);
  cudaFree(c->d_qeff); cudaFree(c->d_olat); cudaFree(c->d_low); cudaFree(c->d_out);
  cudaFree(c->d_part_m); cudaFree(c->d_part_l); cudaFree(c->d_part_o);
  cudaFree(c->d_plan); cudaFree(c->d_status);
  if (c->h_status) cudaFreeHost(c->h_status);
  if (c->h_plan) cudaFreeHost(c->h_plan);
  if (c->plan_ev) cudaEventDestroy(c->plan_ev);
  if (c->plan_ev_b) cudaEventDestroy(c->plan_ev_b);
  if (c->fwd_ev) cudaEventDestroy(c->fwd_ev);
  if (c->copy_stream) cudaStreamDestroy(c->copy_stream);
  if (c->h_pinned) cudaFreeHost(c->h_pinned);
  for (auto& es : c->ev_pool)
    for (auto& e : es.ev) cudaEventDestroy(e);
  delete c;
}

int fst_cuda_mla_set_stream(FstMlaCtx* c, void* s) {
  if (!c) return fail(FST_MLA_ERR_ARG, "null context");
  CU(cudaStreamSynchronize(c->stream));
  c->stream = (cudaStream_t)s;
  return FST_MLA_OK;
}

int fst_cuda_mla_sync(FstMlaCtx* c) {
  if (!c) return fail(FST_MLA_ERR_ARG, "null context");
  // The status word rides the stream (a blocking copy after the synchronisation costs ~10 us more) --
  // or, behind a whole layer call, was stored to h_status by the last GEMM itself if it was not
  // zero (GemmArgs::status_host), which saves the copy and its 8 us of completion latency.
  if (!c->status_by_kernel)
    CU(cudaMemcpyAsync(c->h_status, c->d_status, sizeof(int), cudaMemcpyDeviceToHost, c->stream));
  c->status_by_kernel = false;
  CU(cudaStreamSynchronize(c->stream));
  const int st = *reinterpret_cast<volatile int*>(c->h_status);
  if (st != 0) {
    *c->h_status = 0;
    cudaMemset(c->d_status, 0, sizeof(int));
    return fail(FST_MLA_ERR_DEVICE_CHECK, "a kernel gave up a bounded wait (status %d)", st);
  }
  return FST_MLA_OK;
}

int fst_cuda_mla_set_layer_weights(FstMlaCtx* c, int lid, const FstMlaWeights* w) {
  if (!c || !w) return fail(FST_MLA_ERR_ARG, "null argument");
  if (lid < 0 || lid >= c->cfg.n_layers) return fail(FST_MLA_ERR_ARG, "layer %d out of range", lid);
  const Dims& d = c->d;
  const bool need_b = !d.v4;
  if (!w->wq_a || !w->wq_b || !w->wkv_a || !w->wo_b || (need_b && !w->wkv_b) || (d.v4 && !w->wo_a))
    return fail(FST_MLA_ERR_ARG, "a weight matrix this preset needs is NULL");
  CU(cudaSetDevice(c->cfg.device));
  LayerW& L = c->layers[lid];
  auto up = [&](bf16** dst, const uint16_t* src, size_t n) -> int {
    if (!*dst) {
      int rc = dev_alloc(dst, n);
      if (rc) return rc;
    }
    CU(cudaMemcpy(*dst, src, n * sizeof(bf16), cudaMemcpyHostToDevice));
    return FST_MLA_OK;
  };
  int rc;
  // [wq_a; wkv_a] stacked so that both compressions are one GEMM over h
  if (!L.w_cmp && (rc = dev_alloc(&L.w_cmp, (size_t)d.cmp_n * d.hidden))) return rc;
  CU(cudaMemcpy(L.w_cmp, w->wq_a, (size_t)d.q_lora * d.hidden * 2, cudaMemcpyHostToDevice));
  CU(cudaMemcpy(L.w_cmp + (size_t)d.q_lora * d.hidden, w->wkv_a, (size_t)d.row * d.hidden * 2, cudaMemcpyHostToDevice));
  if ((rc = up(&L.wq_b, w->wq_b, (size_t)d.H * d.q_head * d.q_lora))) return rc;
  if (need_b && (rc = up(&L.wkv_b, w->wkv_b, (size_t)d.H * (d.nope + d.v_head) * d.kv_lora))) return rc;
  if (d.v4 && (rc = up(&L.wo_a, w->wo_a, (size_t)d.low * (d.H * d.d_v / c->cfg.o_groups)))) return rc;
  if ((rc = up(&L.wo_b, w->wo_b, (size_t)d.hidden * d.low))) return rc;
  if (w->q_norm) {
    if ((rc = up(&L.q_norm, w->q_norm, d.q_lora))) return rc;
  } else if (L.q_norm) {
    cudaFree(L.q_norm);
    L.q_norm = nullptr;
  }
  if (w->kv_norm) {
    if ((rc = up(&L.kv_norm, w->kv_norm, d.kv_lora))) return rc;
  } else if (L.kv_norm) {
    cudaFree(L.kv_norm);
    L.kv_norm = nullptr;
  }
  if (w->attn_norm) {
    if ((rc = up(&L.attn_norm, w->attn_norm, d.hidden))) return rc;
  } else if (L.attn_norm) {
    cudaFree(L.attn_norm);
    L.attn_norm = nullptr;
  }
  if (d.v4) {
    if (!L.sinks && (rc = dev_alloc(&L.sinks, (size_t)d.H))) return rc;
    if (w->attn_sinks)
      CU(cudaMemcpy(L.sinks, w->attn_sinks, d.H * sizeof(float), cudaMemcpyHostToDevice));
    else
      CU(cudaMemset(L.sinks, 0, d.H * sizeof(float)));  // empty sinks: logit 0 (reference 3623)
  }
  L.set = true;
  return FST_MLA_OK;
}

int fst_cuda_mla_set_rope_theta(FstMlaCtx* c, float theta) {
  if (!c) return fail(FST_MLA_ERR_ARG, "null context");
  if (!(theta > 0.0f) || !std::isfinite(theta)) return fail(FST_MLA_ERR_ARG, "rope_theta must be positive");
  if (theta != c->cfg.rope_theta) {
    c->cfg.rope_theta = theta;
    for (auto& t : c->lut_tag) t.clear();  // the cached table rows were built with the old base
    c->planned = false;
  }
  return FST_MLA_OK;
}

int fst_cuda_mla_set_layer_rope(FstMlaCtx* c, int lid, int32_t yarn) {
  if (!c) return fail(FST_MLA_ERR_ARG, "null context");
  if (lid < 0 || lid >= c->cfg.n_layers) return fail(FST_MLA_ERR_ARG, "layer %d out of range", lid);
  if (yarn != 0 && yarn != 1) return fail(FST_MLA_ERR_ARG, "RoPE kind %d (0: plain, 1: YaRN)", yarn);
  if (c->layer_yarn[lid] != yarn) {
    c->layer_yarn[lid] = (int8_t)yarn;
    c->planned = false;  // the next plan uploads the tables of every kind in use
  }
  return FST_MLA_OK;
}

int fst_cuda_mla_set_layer_draft_form(FstMlaCtx* c, int lid, int32_t on) {
  if (!c) return fail(FST_MLA_ERR_ARG, "null context");
  if (lid < 0 || lid >= c->cfg.n_layers) return fail(FST_MLA_ERR_ARG, "layer %d out of range", lid);
  if (on && !c->d.v4) return fail(FST_MLA_ERR_ARG, "the draft model's layer has the V4 form (512-wide rows)");
  c->layers[lid].draft_form = on != 0;
  return FST_MLA_OK;
}

int fst_cuda_mla_set_layer_compressor(FstMlaCtx* c, int lid, const FstMlaCompressor* w) {
  if (!c) return fail(FST_MLA_ERR_ARG, "null context");
  if (lid < 0 || lid >= c->cfg.n_layers) return fail(FST_MLA_ERR_ARG, "layer %d out of range", lid);
  if (!c->d.v4) return fail(FST_MLA_ERR_ARG, "the KV compressor belongs to the V4 form (512-wide rows)");
  const int ratio = w ? w->ratio : 0;
  if (ratio != 0 && ratio != 4 && ratio != 128) return fail(FST_MLA_ERR_ARG, "compress ratio %d (0, 4 or 128)", ratio);
  if (ratio && (!w->wkv || !w->wgate || !w->ape || !w->norm)) return fail(FST_MLA_ERR_ARG, "a compressor tensor is NULL");
  for (int s = 0; s < c->cfg.max_seqs; ++s)
    if (c->live[s] && c->lens[s] > 0)
      return fail(FST_MLA_ERR_STATE, "set the compressors before any sequence holds rows");
  CU(cudaSetDevice(c->cfg.device));
  LayerW& L = c->layers[lid];
  cudaFree(L.w_cmp_proj); cudaFree(L.cmp_ape); cudaFree(L.cmp_norm); cudaFree(L.cmp_state); cudaFree(L.cmp_snap);
  L.w_cmp_proj = nullptr; L.cmp_ape = nullptr; L.cmp_norm = nullptr; L.cmp_state = nullptr; L.cmp_snap = nullptr;
  L.cmp_ratio = ratio;
  if (ratio) {
    const Dims& d = c->d;
    const size_t width = cmp_width(c, ratio), slot = cmp_slot_floats(c, ratio);
    int rc = dev_alloc(&L.w_cmp_proj, 2 * width * d.hidden);
    if (!rc) rc = dev_alloc(&L.cmp_ape, (size_t)ratio * width);
    if (!rc) rc = dev_alloc(&L.cmp_norm, (size_t)d.kv_lora);
    if (!rc) rc = dev_alloc(&L.cmp_state, slot * c->cfg.max_seqs);
    if (rc) return rc;
    CU(cudaMemcpy(L.w_cmp_proj, w->wkv, width * d.hidden * 2, cudaMemcpyHostToDevice));
    CU(cudaMemcpy(L.w_cmp_proj + width * d.hidden, w->wgate, width * d.hidden * 2, cudaMemcpyHostToDevice));
    CU(cudaMemcpy(L.cmp_ape, w->ape, (size_t)ratio * width * sizeof(float), cudaMemcpyHostToDevice));
    CU(cudaMemcpy(L.cmp_norm, w->norm, (size_t)d.kv_lora * 2, cudaMemcpyHostToDevice));
    CU(cudaMemset(L.cmp_state, 0, slot * c->cfg.max_seqs * sizeof(float)));
    L.cmp_pos.assign(c->cfg.max_seqs, 0);
    L.cmp_pos_snap.assign(c->cfg.max_seqs, 0);
  }
  c->has_cmp = false;
  c->cmp_min_ratio = 0;
  for (const LayerW& l : c->layers)
    if (l.cmp_ratio) {
      c->has_cmp = true;
      c->cmp_min_ratio = c->cmp_min_ratio ? std::min(c->cmp_min_ratio, l.cmp_ratio) : l.cmp_ratio;
    }
  c->planned = false;
  return FST_MLA_OK;
}

int fst_cuda_mla_seq_snapshot(FstMlaCtx* c, int32_t seq) {
  if (!c) return fail(FST_MLA_ERR_ARG, "null context");
  if (!seq_ok(c, seq)) return fail(FST_MLA_ERR_ARG, "sequence %d is not allocated", seq);
  CU(cudaSetDevice(c->cfg.device));
  for (LayerW& l : c->layers)
    if (l.cmp_ratio) {
      const size_t n = cmp_slot_floats(c, l.cmp_ratio);
      if (!l.cmp_snap) {
        int rc = dev_alloc(&l.cmp_snap, n * c->cfg.max_seqs);
        if (rc) return rc;
      }
      CU(cudaMemcpyAsync(l.cmp_snap + (size_t)seq * n, l.cmp_state + (size_t)seq * n, n * sizeof(float),
                         cudaMemcpyDeviceToDevice, c->stream));
      l.cmp_pos_snap[seq] = l.cmp_pos[seq];
    }
  c->snap_len[seq] = c->lens[seq];
  return FST_MLA_OK;
}

int fst_cuda_mla_cmp_read(FstMlaCtx* c, int lid, int32_t seq, uint16_t* rows, int32_t cap, int32_t* n_out) {
  if (!c || !n_out) return fail(FST_MLA_ERR_ARG, "null argument");
  if (lid < 0 || lid >= c->cfg.n_layers) return fail(FST_MLA_ERR_ARG, "layer %d out of range", lid);
  if (!seq_ok(c, seq)) return fail(FST_MLA_ERR_ARG, "sequence %d is not allocated", seq);
  const LayerW& L = c->layers[lid];
  const int n = L.cmp_ratio ? L.cmp_pos[seq] / L.cmp_ratio : 0;
  *n_out = n;
  if (!rows) return FST_MLA_OK;
  if (cap < n) return fail(FST_MLA_ERR_ARG, "%d compressed rows, room for %d", n, cap);
  CU(cudaSetDevice(c->cfg.device));
  const int pt = c->cfg.page_tokens, row = c->d.row;
  for (int r = 0; r < n; ++r) {
    const bf16* src = c->pools[lid] + ((long long)c->comp_tables[seq][r / pt] * pt + r % pt) * row;
    CU(cudaMemcpyAsync(rows + (size_t)r * row, src, (size_t)row * 2, cudaMemcpyDeviceToHost, c->stream));
  }
  CU(cudaStreamSynchronize(c->stream));
  return FST_MLA_OK;
}

/* ---- paged cache ---------------------------------------------------------------------- */
int fst_cuda_mla_seq_alloc(FstMlaCtx* c, int32_t* seq_out) {
  if (!c || !seq_out) return fail(FST_MLA_ERR_ARG, "null argument");
  if (c->free_seqs.empty()) return fail(FST_MLA_ERR_CAPACITY, "all %d sequence slots are in use", c->cfg.max_seqs);
  int s = c->free_seqs.back();
  c->free_seqs.pop_back();
  c->live[s] = 1;
  c->lens[s] = 0;
  c->tables[s].clear();
  c->comp_tables[s].clear();
  c->snap_len[s] = -1;
  if (c->has_cmp) {
    // a new sequence starts with an empty compressor window (reset_compressor_state, reference 3160-3169)
    CU(cudaSetDevice(c->cfg.device));
    for (LayerW& l : c->layers)
      if (l.cmp_ratio) {
        const size_t n = cmp_slot_floats(c, l.cmp_ratio);
        CU(cudaMemsetAsync(l.cmp_state + (size_t)s * n, 0, n * sizeof(float), c->stream));
        l.cmp_pos[s] = 0;
      }
  }
  *seq_out = s;
  c->planned = false;
  return FST_MLA_OK;
}

int fst_cuda_mla_seq_truncate(FstMlaCtx* c, int32_t seq, int32_t n_tokens) {
  if (!c) return fail(FST_MLA_ERR_ARG, "null context");
  if (!seq_ok(c, seq)) return fail(FST_MLA_ERR_ARG, "sequence %d is not allocated", seq);
  if (n_tokens < 0 || n_tokens > c->lens[seq])
    return fail(FST_MLA_ERR_ARG, "truncate to %d outside [0, %d]", n_tokens, c->lens[seq]);
  CU(cudaSetDevice(c->cfg.device));
  // zero the dropped rows in every layer, as the reference rollback does (6132-6147)
  const int n_drop = c->lens[seq] - n_tokens;
  if (n_drop > 0) {
    std::vector<long long> offs(n_drop);
    for (int i = 0; i < n_drop; ++i) offs[i] = row_offset(c, seq, n_tokens + i);
    long long* d_offs = nullptr;
    CU(cudaMalloc((void**)&d_offs, n_drop * sizeof(long long)));
    cudaError_t e = cudaMemcpyAsync(d_offs, offs.data(), n_drop * sizeof(long long), cudaMemcpyHostToDevice, c->stream);
    for (int l = 0; l < c->cfg.n_layers && e == cudaSuccess; ++l) {
      launch_zero_rows(c->pools[l], d_offs, n_drop, c->d.row, c->stream);
      c->launches += 1;
    }
    if (e == cudaSuccess) e = cudaStreamSynchronize(c->stream);
    cudaFree(d_offs);
    if (e != cudaSuccess) return fail(FST_MLA_ERR_CUDA, "rollback failed: %s", cudaGetErrorString(e));
  }
  const size_t keep = ((size_t)n_tokens + c->cfg.page_tokens - 1) / c->cfg.page_tokens;
  auto& t = c->tables[seq];
  while (t.size() > keep) {
    c->free_pages.push_back(t.back());
    t.pop_back();
  }
  if (c->has_cmp) {
    // The compressed rows emitted by the dropped rows go with them.  The window state comes back
    // from the snapshot taken at this length (the reference restores cmp_snap, 6149-6152); without
    // one the state keeps what the dropped rows wrote, which only a truncation to 0 makes harmless.
    const size_t keep_c = ((size_t)(n_tokens / c->cmp_min_ratio) + c->cfg.page_tokens - 1) / c->cfg.page_tokens;
    auto& ct = c->comp_tables[seq];
    while (ct.size() > keep_c) {
      c->free_pages.push_back(ct.back());
      ct.pop_back();
    }
    const bool restore = c->snap_len[seq] == n_tokens;
    for (LayerW& l : c->layers)
      if (l.cmp_ratio && l.cmp_pos[seq] > n_tokens) {
        const size_t n = cmp_slot_floats(c, l.cmp_ratio);
        if (restore && l.cmp_snap) {
          CU(cudaMemcpyAsync(l.cmp_state + (size_t)seq * n, l.cmp_snap + (size_t)seq * n, n * sizeof(float),
                             cudaMemcpyDeviceToDevice, c->stream));
          l.cmp_pos[seq] = l.cmp_pos_snap[seq];
        } else {
          if (n_tokens == 0) CU(cudaMemsetAsync(l.cmp_state + (size_t)seq * n, 0, n * sizeof(float), c->stream));
          l.cmp_pos[seq] = n_tokens;
        }
      }
    if (n_tokens < c->snap_len[seq]) c->snap_len[seq] = -1;
  }
  c->lens[seq] = n_tokens;
  c->planned = false;
  return FST_MLA_OK;
}

int fst_cuda_mla_seq_free(FstMlaCtx* c, int32_t seq) {
  int rc = fst_cuda_mla_seq_truncate(c, seq, 0);
  if (rc) return rc;
  c->live[seq] = 0;
  c->free_seqs.push_back(seq);
  return FST_MLA_OK;
}

int fst_cuda_mla_seq_reserve(FstMlaCtx* c, int32_t seq, int32_t n_tokens) {
  if (!c) return fail(FST_MLA_ERR_ARG, "null context");
  if (!seq_ok(c, seq)) return fail(FST_MLA_ERR_ARG, "sequence %d is not allocated", seq);
  if (n_tokens < 0) return fail(FST_MLA_ERR_ARG, "negative length");
  c->planned = false;
  return reserve_pages(c, seq, n_tokens);
}

int fst_cuda_mla_seq_len(FstMlaCtx* c, int32_t seq, int32_t* len_out) {
  if (!c || !len_out) return fail(FST_MLA_ERR_ARG, "null argument");
  if (!seq_ok(c, seq)) return fail(FST_MLA_ERR_ARG, "sequence %d is not allocated", seq);
  *len_out = c->lens[seq];
  return FST_MLA_OK;
}

int fst_cuda_mla_reset(FstMlaCtx* c) {
  if (!c) return fail(FST_MLA_ERR_ARG, "null context");
  CU(cudaSetDevice(c->cfg.device));
  CU(cudaStreamSynchronize(c->stream));
  c->free_pages.clear();
  c->free_seqs.clear();
  for (int i = c->cfg.n_pages - 1; i >= 0; --i) c->free_pages.push_back(i);
  for (int i = c->cfg.max_seqs - 1; i >= 0; --i) c->free_seqs.push_back(i);
  for (auto& t : c->tables) t.clear();
  for (auto& t : c->comp_tables) t.clear();
  std::fill(c->snap_len.begin(), c->snap_len.end(), -1);
  for (LayerW& l : c->layers)
    if (l.cmp_ratio) {
      CU(cudaMemsetAsync(l.cmp_state, 0, cmp_slot_floats(c, l.cmp_ratio) * c->cfg.max_seqs * sizeof(float), c->stream));
      std::fill(l.cmp_pos.begin(), l.cmp_pos.end(), 0);
    }
  std::fill(c->lens.begin(), c->lens.end(), 0);
  std::fill(c->live.begin(), c->live.end(), 0);
  const size_t bytes = (size_t)c->cfg.n_pages * c->cfg.page_tokens * c->d.row * sizeof(bf16);
  for (auto p : c->pools) CU(cudaMemsetAsync(p, 0, bytes, c->stream));
  CU(cudaStreamSynchronize(c->stream));
  c->planned = false;
  return FST_MLA_OK;
}

int fst_cuda_mla_block_table(FstMlaCtx* c, int32_t seq, int32_t* out, int32_t cap, int32_t* n_out) {
  if (!c || !n_out) return fail(FST_MLA_ERR_ARG, "null argument");
  if (!seq_ok(c, seq)) return fail(FST_MLA_ERR_ARG, "sequence %d is not allocated", seq);
  const auto& t = c->tables[seq];
  for (size_t i = 0; i < t.size() && (int)i < cap && out; ++i) out[i] = t[i];
  *n_out = (int32_t)t.size();
  return FST_MLA_OK;
}

int fst_cuda_mla_free_pages(FstMlaCtx* c, int32_t* n_out) {
  if (!c || !n_out) return fail(FST_MLA_ERR_ARG, "null argument");
  *n_out = (int32_t)c->free_pages.size();
  return FST_MLA_OK;
}

int fst_cuda_mla_row_offset(FstMlaCtx* c, int32_t seq, int32_t pos, int64_t* off_out) {
  if (!c || !off_out) return fail(FST_MLA_ERR_ARG, "null argument");
  if (!seq_ok(c, seq)) return fail(FST_MLA_ERR_ARG, "sequence %d is not allocated", seq);
  if (pos < 0 || (size_t)pos >= c->tables[seq].size() * c->cfg.page_tokens)
    return fail(FST_MLA_ERR_ARG, "row %d has no page", pos);
  *off_out = row_offset(c, seq, pos);
  return FST_MLA_OK;
}

static int cache_copy(FstMlaCtx* c, int lid, int32_t seq, int32_t pos0, int32_t n, uint16_t* rows, bool write) {
  if (!c || (!rows && n > 0)) return fail(FST_MLA_ERR_ARG, "null argument");
  if (lid < 0 || lid >= c->cfg.n_layers) return fail(FST_MLA_ERR_ARG, "layer %d out of range", lid);
  if (!seq_ok(c, seq)) return fail(FST_MLA_ERR_ARG, "sequence %d is not allocated", seq);
  if (pos0 < 0 || n < 0) return fail(FST_MLA_ERR_ARG, "negative row range");
  CU(cudaSetDevice(c->cfg.device));
  if (write) {
    int rc = reserve_pages(c, seq, pos0 + n);
    if (rc) return rc;
    c->planned = false;
  } else if (pos0 + n > c->lens[seq]) {
    return fail(FST_MLA_ERR_ARG, "rows [%d, %d) beyond the sequence length %d", pos0, pos0 + n, c->lens[seq]);
  }
  const int pt = c->cfg.page_tokens, row = c->d.row;
  int done = 0;
  while (done < n) {  // one copy per page-contiguous run
    const int pos = pos0 + done, run = std::min(n - done, pt - pos % pt);
    bf16* dev = c->pools[lid] + row_offset(c, seq, pos);
    uint16_t* host = rows + (size_t)done * row;
    if (write)
      CU(cudaMemcpyAsync(dev, host, (size_t)run * row * 2, cudaMemcpyHostToDevice, c->stream));
    else
      CU(cudaMemcpyAsync(host, dev, (size_t)run * row * 2, cudaMemcpyDeviceToHost, c->stream));
    done += run;
  }
  CU(cudaStreamSynchronize(c->stream));
  return FST_MLA_OK;
}

int fst_cuda_mla_cache_write(FstMlaCtx* c, int lid, int32_t seq, int32_t pos0, int32_t n, const uint16_t* rows) {
  return cache_copy(c, lid, seq, pos0, n, const_cast<uint16_t*>(rows), true);
}
int fst_cuda_mla_cache_read(FstMlaCtx* c, int lid, int32_t seq, int32_t pos0, int32_t n, uint16_t* rows) {
  return cache_copy(c, lid, seq, pos0, n, rows, false);
}

int fst_cuda_mla_pool_read(FstMlaCtx* c, int lid, uint16_t* out, size_t bytes) {
  if (!c || !out) return fail(FST_MLA_ERR_ARG, "null argument");
  if (lid < 0 || lid >= c->cfg.n_layers) return fail(FST_MLA_ERR_ARG, "layer %d out of range", lid);
  const size_t full = (size_t)c->cfg.n_pages * c->cfg.page_tokens * c->d.row * 2;
  if (bytes > full) return fail(FST_MLA_ERR_ARG, "pool holds %zu bytes", full);
  CU(cudaSetDevice(c->cfg.device));
  CU(cudaStreamSynchronize(c->stream));
  CU(cudaMemcpy(out, c->pools[lid], bytes, cudaMemcpyDeviceToHost));
  return FST_MLA_OK;
}

/* ---- planning ------------------------------------------------------------------------- */
}  // extern "C"

namespace {

// A plan has two parts.  The first is per token: RoPE rows and the addresses of the appended rows
// -- all that the kernels in front of the attention need.  The second is the split-KV schedule
// with the block tables.  fst_cuda_mla_forward uploads the first, launches the front kernels and
// builds the second while they run; fst_cuda_mla_plan does both at once with one copy.
// *reused: the valid plan answers the request, nothing was built.
int plan_tokens_part(FstMlaCtx* c, const FstMlaSeqStep* steps, int32_t n_seqs, int32_t causal, bool upload_now,
                     bool* reused) {
  *reused = false;
  if (!c || (!steps && n_seqs > 0)) return fail(FST_MLA_ERR_ARG, "null argument");
  if (n_seqs < 0) return fail(FST_MLA_ERR_ARG, "negative sequence count");
  const Dims& d = c->d;
  // The same steps on unchanged sequences (anything that touches a sequence clears `planned`):
  // the plan on the device is still the right one -- layers 2 .. L of a model step.
  if (c->planned && c->plan_reuse && causal == c->last_causal && (size_t)n_seqs == c->last_steps.size() &&
      (n_seqs == 0 || memcmp(steps, c->last_steps.data(), (size_t)n_seqs * sizeof(FstMlaSeqStep)) == 0)) {
    ++c->plans_reused;
    *reused = true;
    return FST_MLA_OK;
  }
  c->planned = false;
  long long T = 0;
  for (int b = 0; b < n_seqs; ++b) {
    const FstMlaSeqStep& s = steps[b];
    if (!seq_ok(c, s.seq)) return fail(FST_MLA_ERR_ARG, "step %d: sequence %d is not allocated", b, s.seq);
    if (s.pos0 < 0 || s.q_len < 0) return fail(FST_MLA_ERR_ARG, "step %d: negative position or length", b);
    for (int b2 = 0; b2 < b; ++b2)
      if (steps[b2].seq == s.seq) return fail(FST_MLA_ERR_ARG, "sequence %d appears twice", s.seq);
    T += s.q_len;
  }
  if (T > c->cfg.max_tokens)
    return fail(FST_MLA_ERR_CAPACITY, "%lld new tokens exceed max_tokens %d", T, c->cfg.max_tokens);
  CU(cudaSetDevice(c->cfg.device));
  // reserve pages first so that a failure leaves no half-built plan (the reference asserts
  // seq_pos_ + M <= max_seq, src/fst_engine.cpp:3327)
  for (int b = 0; b < n_seqs; ++b) {
    const FstMlaSeqStep& s = steps[b];
    const int need = s.append ? s.pos0 + s.q_len : s.pos0;
    if (!s.append && need > c->lens[s.seq])
      return fail(FST_MLA_ERR_ARG, "step %d: rows [0, %d) are not all cached (length %d)", b, need, c->lens[s.seq]);
    if (s.append) {
      int rc = reserve_pages(c, s.seq, need);
      if (rc) return rc;
    }
  }

  bool need[2];
  rope_kinds(c, need);
  std::vector<long long>& dst = c->pl_dst;
  std::vector<int32_t>&tok_table = c->pl_tok_table, &tables = c->pl_tables, &kvlen = c->pl_kvlen, &kvlo = c->pl_kvlo;
  for (int k = 0; k < 2; ++k) c->pl_lut[k].resize(need[k] ? (size_t)T * d.rope : 0);
  dst.resize(T);
  tok_table.resize(T);
  c->pl_tok_ctable.resize(T);
  c->pl_tok_step.resize(T);
  kvlen.resize(T);
  kvlo.resize(T);
  tables.clear();
  int t = 0;
  for (int b = 0; b < n_seqs; ++b) {
    const FstMlaSeqStep& s = steps[b];
    const int toff = (int)tables.size();
    tables.insert(tables.end(), c->tables[s.seq].begin(), c->tables[s.seq].end());
    const int ctoff = (int)tables.size();  // the pages of the sequence's compressed rows
    tables.insert(tables.end(), c->comp_tables[s.seq].begin(), c->comp_tables[s.seq].end());
    const int rp0 = s.rope_pos0 >= 0 ? s.rope_pos0 : s.pos0;
    for (int i = 0; i < s.q_len; ++i, ++t) {
      c->pl_tok_ctable[t] = ctoff;
      c->pl_tok_step[t] = b;
      for (int k = 0; k < 2; ++k)
        if (need[k]) memcpy(&c->pl_lut[k][(size_t)t * d.rope], lut_row_cached(c, k, rp0 + i), (size_t)d.rope * sizeof(float));
      dst[t] = s.append ? row_offset(c, s.seq, s.pos0 + i) : -1;
      tok_table[t] = toff;
      int len = s.append ? s.pos0 + s.q_len : s.pos0;
      if (causal && s.append) len = std::min(len, s.pos0 + i + 1);  // drop s > seq_pos_ + m (3626)
      kvlen[t] = len;
      // sliding window (the draft model's attention, src/fst_engine.cpp:2534-2576 keeps the last
      // `window_size` rows in a ring): the last `window` rows of what the token may see
      kvlo[t] = s.window > 0 ? std::max(0, len - s.window) : 0;
    }
  }
  if ((int)tables.size() > c->tables_cap) return fail(FST_MLA_ERR_CAPACITY, "block tables overflow");
  c->pl_steps.assign(steps, steps + n_seqs);
  c->pl_causal = causal;
  c->T = (int)T;

  // the first part of the pinned blob (once the previous plan's copies have left it)
  CU(cudaEventSynchronize(c->plan_ev));
  CU(cudaEventSynchronize(c->plan_ev_b));
  size_t off = 0;
  auto put = [&](const void* src, size_t bytes) -> unsigned char* {
    unsigned char* dev = c->d_plan + off;
    if (bytes) memcpy(c->h_plan + off, src, bytes);
    off = (off + bytes + 255) & ~(size_t)255;
    return dev;
  };
  for (int k = 0; k < 2; ++k)
    c->d_lut_k[k] = need[k] ? reinterpret_cast<float*>(put(c->pl_lut[k].data(), c->pl_lut[k].size() * sizeof(float))) : nullptr;
  c->d_dst = reinterpret_cast<long long*>(put(dst.data(), (size_t)T * sizeof(long long)));
  // what the compressor kernels read, per class of compressed layers present
  for (int k = 1; k < N_CLASSES; ++k) {
    Sched& S = c->sched[k];
    S.d_ctoks = nullptr;
    S.n_csteps = 0;
    bool present = false;
    int kind = 0;
    for (int l = 0; l < c->cfg.n_layers; ++l)
      if (c->layers[l].cmp_ratio == CLASS_RATIO[k]) {
        present = true;
        kind = c->layer_yarn[l] ? 1 : 0;
      }
    if (!present) continue;
    const int ratio = CLASS_RATIO[k], pt = c->cfg.page_tokens;
    std::vector<CompressTok> ctoks(T);
    std::vector<CompressStep> csteps;
    std::vector<float> lut_cmp((size_t)T * d.rope, 0.0f);
    int tt = 0;
    for (int b = 0; b < n_seqs; ++b) {
      const FstMlaSeqStep& st = steps[b];
      if (st.q_len > 0) csteps.push_back(CompressStep{tt, st.q_len, st.seq, 0});
      for (int i = 0; i < st.q_len; ++i, ++tt) {
        const int pos = st.pos0 + i;
        ctoks[tt] = CompressTok{-1, pos, 0};
        if (st.append && (pos + 1) % ratio == 0) {
          // compressed row number (pos + 1) / ratio - 1, rotated at position pos + 1 - ratio (3252-3254)
          const int cr = (pos + 1) / ratio - 1;
          ctoks[tt].dst = ((long long)c->comp_tables[st.seq][cr / pt] * pt + cr % pt) * d.row;
          memcpy(&lut_cmp[(size_t)tt * d.rope], lut_row_cached(c, kind, pos + 1 - ratio), (size_t)d.rope * sizeof(float));
        }
      }
    }
    S.d_ctoks = reinterpret_cast<CompressTok*>(put(ctoks.data(), ctoks.size() * sizeof(CompressTok)));
    S.d_csteps = reinterpret_cast<CompressStep*>(put(csteps.data(), csteps.size() * sizeof(CompressStep)));
    S.d_lut_cmp = reinterpret_cast<float*>(put(lut_cmp.data(), lut_cmp.size() * sizeof(float)));
    S.n_csteps = (int)csteps.size();
  }
  if (off > c->plan_cap) return fail(FST_MLA_ERR_CAPACITY, "plan blob overflow");
  c->pl_off_b = off;
  c->front_uploaded = upload_now && off > 0;
  if (c->front_uploaded) {
    CU(cudaMemcpyAsync(c->d_plan, c->h_plan, off, cudaMemcpyHostToDevice, c->stream));
    CU(cudaEventRecord(c->plan_ev, c->stream));
  }
  return FST_MLA_OK;
}

// One stream of cache tiles in the schedule: a query token's raw rows [lo, hi) of the table that
// starts at `table`, or its visible compressed rows.  A token's streams are adjacent.
struct TileStream {
  int32_t tok, table, lo, hi;
};

// The split-KV schedule of one layer class.  The concatenated tiles of all streams are cut into
// n_ctas contiguous runs of about equal COST; a run that crosses a stream boundary yields one segment
// (and one partial) per stream it touches.  The unit is a cache page where pages hold 64 tokens,
// else ATTN_TILE rows.  Cost, in half units: 2 per tile plus SEG_COST2 per segment -- a segment
// pays for its Q_eff block (one ring slot), refilling the pipeline and writing its partial
// (measured inside the pipelined layer: about three 64-token tiles of the streaming kernel).
void cut_schedule(const FstMlaCtx* c, const std::vector<TileStream>& streams, int T, std::vector<AttnSeg>* segs_out,
                  std::vector<int32_t>* cta_seg_out, std::vector<int32_t>* tok_part_out, long long* kv_rows_out,
                  int max_ctas = 0) {
  const int unit = c->cfg.page_tokens == 64 ? 64 : ATTN_TILE;
  const long long SEG_COST2 = unit == 64 ? 6 : 5;
  const int n_streams = (int)streams.size();
  long long total_tiles = 0, kv_rows = 0, n_nonempty = 0;
  // tiles are counted from the tile that holds the first visible row
  auto tile0_of = [&](int i) { return streams[i].lo / unit; };
  auto tiles_of = [&](int i) { return (streams[i].hi + unit - 1) / unit - tile0_of(i); };
  for (int i = 0; i < n_streams; ++i) {
    total_tiles += tiles_of(i);
    kv_rows += streams[i].hi - streams[i].lo;
    n_nonempty += streams[i].hi > 0;
  }
  const int n_ctas = (int)std::min<long long>(max_ctas > 0 ? max_ctas : c->n_sm, std::max<long long>(total_tiles, 1));
  std::vector<AttnSeg>& segs = *segs_out;
  std::vector<int32_t>& cta_seg = *cta_seg_out;
  std::vector<int32_t> parts_of(T, 0);
  segs.clear();
  cta_seg.assign(n_ctas + 1, 0);
  int st = 0, tile_in = 0, part = 0;
  auto skip_empty = [&]() {
    while (st < n_streams && tile_in >= tiles_of(st)) {
      ++st;
      tile_in = 0;
    }
  };
  skip_empty();
  long long tiles_left = total_tiles, streams_left = n_nonempty;  // streams not yet started
  for (int k = 0; k < n_ctas; ++k) {
    cta_seg[k] = (int)segs.size();
    const bool last = k == n_ctas - 1;
    // what is left, shared equally among the CTAs that are left: the tiles, a segment for every
    // stream still to start (and for the one this CTA resumes), and one more segment for every
    // later CTA, which will most likely resume a stream
    const long long mid = tile_in > 0 ? 1 : 0;
    const long long left2 = 2 * tiles_left + SEG_COST2 * (streams_left + mid + (n_ctas - k - 1));
    long long budget2 = left2 / (n_ctas - k);
    while (st < n_streams) {
      long long room = last ? (1ll << 40) : (budget2 - SEG_COST2) / 2;  // tiles that still fit
      if (room < 1) {
        if (cta_seg[k] != (int)segs.size()) break;
        room = 1;  // every CTA takes at least one tile
      }
      const TileStream& ts = streams[st];
      const int take = (int)std::min<long long>(room, tiles_of(st) - tile_in);
      AttnSeg sg;
      sg.tok = ts.tok;
      sg.kv_begin = std::max(ts.lo, (tile0_of(st) + tile_in) * unit);  // unaligned only at a window's edge
      sg.kv_end = std::min(ts.hi, (tile0_of(st) + tile_in + take) * unit);
      sg.part = part++;
      sg.table = ts.table;
      segs.push_back(sg);
      parts_of[ts.tok] += 1;
      if (tile_in == 0) --streams_left;
      tile_in += take;
      tiles_left -= take;
      budget2 -= SEG_COST2 + 2 * take;
      skip_empty();
    }
  }
  cta_seg[n_ctas] = (int)segs.size();
  // a token's streams are adjacent and segments are numbered in stream order: its partials are
  // the contiguous range [tok_part[t], tok_part[t + 1])
  tok_part_out->assign(T + 1, 0);
  for (int t = 0; t < T; ++t) (*tok_part_out)[t + 1] = (*tok_part_out)[t] + parts_of[t];
  *kv_rows_out = kv_rows;
}

// The schedule for BLOCKS of query tokens (speculative verify, prefill chunks over a long context:
// every sequence of the call brings the same number G >= 4 of new tokens, which all attend to the
// same rows but for the causal edge).  Cutting token after token would let the G tokens of a
// sequence walk its pages at G different times, and each page would come from HBM G times (measured:
// 13 x the cache bytes for 16-token blocks, L2 hit rate 29 %).  Here the thread blocks form
// n_sm / G GROUPS of G lanes; the sequences' page columns are cut into one run per group exactly as
// the token schedule cuts tiles; lane i of a group walks its group's run for token i of each
// sequence, so the G lanes read the same page at about the same time and it crosses the HBM
// interface once.  Returns false (nothing written) when the call is not of that shape.
bool cut_block_schedule(const FstMlaCtx* c, int T, std::vector<AttnSeg>* segs_out, std::vector<int32_t>* cta_seg_out,
                        std::vector<int32_t>* tok_part_out, long long* kv_rows_out) {
  const int unit = 64;
  if (c->cfg.page_tokens != unit) return false;
  int G = 0, n_seq = 0;
  for (const FstMlaSeqStep& st : c->pl_steps) {
    if (st.q_len == 0) continue;
    if (G && st.q_len != G) return false;
    G = st.q_len;
    ++n_seq;
  }
  if (G < 4 || G > c->n_sm) return false;
  for (int t = 0; t < T; ++t)
    if (c->pl_kvlo[t] != 0) return false;  // sliding windows keep the token schedule
  const int n_groups = c->n_sm / G;
  // one stream per sequence: the rows its last token sees (the tokens of a step are adjacent)
  std::vector<TileStream> cols;
  long long kv_rows = 0, n_cols = 0;
  for (int t0 = 0; t0 < T; t0 += G) {
    int hi = 0;
    for (int i = 0; i < G; ++i) {
      hi = std::max(hi, c->pl_kvlen[t0 + i]);
      kv_rows += c->pl_kvlen[t0 + i];
    }
    cols.push_back(TileStream{t0, c->pl_tok_table[t0], 0, hi});
    n_cols += (hi + unit - 1) / unit;
  }
  if (n_cols < 2ll * n_groups) return false;  // too little work per group to cut it this way
  std::vector<AttnSeg> gsegs;
  std::vector<int32_t> g_seg, unused;
  long long unused_rows = 0;
  cut_schedule(c, cols, T, &gsegs, &g_seg, &unused, &unused_rows, n_groups);
  const int groups = (int)g_seg.size() - 1;
  std::vector<AttnSeg>& segs = *segs_out;
  segs.clear();
  cta_seg_out->assign((size_t)groups * G + 1, 0);
  std::vector<int32_t> parts_of(T, 0);
  for (int g = 0; g < groups; ++g)
    for (int i = 0; i < G; ++i) {
      (*cta_seg_out)[g * G + i] = (int)segs.size();
      for (int k = g_seg[g]; k < g_seg[g + 1]; ++k) {
        const int t = gsegs[k].tok + i;
        AttnSeg sg = gsegs[k];
        sg.tok = t;
        sg.table = c->pl_tok_table[t];
        sg.kv_end = std::min(sg.kv_end, c->pl_kvlen[t]);
        if (sg.kv_end <= sg.kv_begin) continue;  // the causal edge: this token does not reach the run
        sg.part = parts_of[t]++;                   // for now the index among the token's parts
        segs.push_back(sg);
      }
    }
  (*cta_seg_out)[(size_t)groups * G] = (int)segs.size();
  tok_part_out->assign(T + 1, 0);
  for (int t = 0; t < T; ++t) (*tok_part_out)[t + 1] = (*tok_part_out)[t] + parts_of[t];
  // a token's parts ascend with the group index, i.e. with the rows they cover
  for (AttnSeg& sg : segs) sg.part += (*tok_part_out)[sg.tok];
  *kv_rows_out = kv_rows;
  return true;
}

// The second part: schedules (one per layer class in use) and block tables.  on_copy_stream:
// upload it beside the kernels that already run on the context's stream (which then waits for
// it); else one copy of the whole blob (or of the second part, if the first went ahead) on the
// context's stream.
int plan_schedule_part(FstMlaCtx* c, bool on_copy_stream) {
  const int T = c->T;
  std::vector<int32_t>&tok_table = c->pl_tok_table, &tables = c->pl_tables, &kvlen = c->pl_kvlen, &kvlo = c->pl_kvlo;

  // the second part of the pinned blob, behind the first; the device arrays are slices of the
  // device blob
  size_t off = c->pl_off_b;
  auto put = [&](const void* src, size_t bytes) -> unsigned char* {
    unsigned char* dev = c->d_plan + off;
    if (off + bytes <= c->plan_cap && bytes) memcpy(c->h_plan + off, src, bytes);
    off = (off + bytes + 255) & ~(size_t)255;
    return dev;
  };
  bool in_use[N_CLASSES] = {true, false, false};  // class 0 is always built (plan_info, callers without layers)
  for (const LayerW& l : c->layers) in_use[class_of_ratio(l.cmp_ratio)] = true;
  std::vector<TileStream> streams;
  std::vector<AttnSeg> segs;
  std::vector<int32_t> cta_seg, tok_part;
  for (int k = 0; k < N_CLASSES; ++k) {
    Sched& S = c->sched[k];
    S.built = false;
    if (!in_use[k]) continue;
    streams.clear();
    for (int t = 0; t < T; ++t) {
      streams.push_back(TileStream{t, tok_table[t], kvlo[t], kvlen[t]});
      if (k > 0) {
        // compressed row r was emitted at position (r + 1) * ratio - 1 (reference 3630-3635): every
        // row of this call sees all of them in decode, those at or before its own position when
        // causal.  (All rows of the sequence have gone through the compressor when the attention
        // runs: the call's own rows are compressed in front of it.)
        const FstMlaSeqStep& st = c->pl_steps[c->pl_tok_step[t]];
        const int ratio = CLASS_RATIO[k];
        int n_vis = st.append ? (st.pos0 + st.q_len) / ratio : 0;
        if (c->pl_causal) {
          int tok_in_step = t;
          for (int b = 0; b < c->pl_tok_step[t]; ++b) tok_in_step -= c->pl_steps[b].q_len;
          n_vis = std::min(n_vis, (st.pos0 + tok_in_step + 1) / ratio);
        }
        if (n_vis > 0) streams.push_back(TileStream{t, c->pl_tok_ctable[t], 0, n_vis});
      }
    }
    long long kv_rows = 0;
    S.by_blocks = k == 0 && c->block_schedule && cut_block_schedule(c, T, &segs, &cta_seg, &tok_part, &kv_rows);
    if (!S.by_blocks) cut_schedule(c, streams, T, &segs, &cta_seg, &tok_part, &kv_rows);
    if ((int)segs.size() > c->segs_cap || (int)segs.size() > c->max_parts)
      return fail(FST_MLA_ERR_CAPACITY, "split schedule overflow");
    S.d_tok_part = reinterpret_cast<int32_t*>(put(tok_part.data(), (size_t)(T + 1) * sizeof(int32_t)));
    S.d_cta_seg = reinterpret_cast<int32_t*>(put(cta_seg.data(), cta_seg.size() * sizeof(int32_t)));
    S.d_segs = reinterpret_cast<AttnSeg*>(put(segs.data(), segs.size() * sizeof(AttnSeg)));
    S.max_tok_parts = 0;
    S.n_single_part = 0;
    S.min_tok_parts = T > 0 ? (1 << 30) : 0;
    for (int i = 0; i < T; ++i) {
      const int np = tok_part[i + 1] - tok_part[i];
      S.max_tok_parts = std::max(S.max_tok_parts, np);
      S.min_tok_parts = std::min(S.min_tok_parts, np);
      S.n_single_part += np == 1;
    }
    S.n_segs = S.n_parts = (int)segs.size();
    S.n_ctas = (int)cta_seg.size() - 1;
    S.kv_rows = kv_rows;
    S.built = true;
  }
  c->d_tables = reinterpret_cast<int32_t*>(put(tables.data(), tables.size() * sizeof(int32_t)));
  if (off > c->plan_cap) return fail(FST_MLA_ERR_CAPACITY, "plan blob overflow");
  const size_t from = c->front_uploaded ? c->pl_off_b : 0;
  if (on_copy_stream) {
    // beside the front kernels; fwd_ev (recorded when the call began) keeps the copy behind
    // everything that was on the stream before this call and may still read the old tables
    CU(cudaStreamWaitEvent(c->copy_stream, c->fwd_ev, 0));
    CU(cudaMemcpyAsync(c->d_plan + from, c->h_plan + from, off - from, cudaMemcpyHostToDevice, c->copy_stream));
    CU(cudaEventRecord(c->plan_ev_b, c->copy_stream));
    CU(cudaStreamWaitEvent(c->stream, c->plan_ev_b, 0));
  } else {
    CU(cudaMemcpyAsync(c->d_plan + from, c->h_plan + from, off - from, cudaMemcpyHostToDevice, c->stream));
    CU(cudaEventRecord(c->plan_ev, c->stream));
  }
  c->last_steps = c->pl_steps;
  c->last_causal = c->pl_causal;
  ++c->plans_built;
  c->planned = true;
  return FST_MLA_OK;
}

}  // namespace

extern "C" {

int fst_cuda_mla_plan(FstMlaCtx* c, const FstMlaSeqStep* steps, int32_t n_seqs, int32_t causal) {
  bool reused = false;
  int rc = plan_tokens_part(c, steps, n_seqs, causal, false, &reused);
  if (rc || reused) return rc;
  return plan_schedule_part(c, false);
}

int fst_cuda_mla_set_plan_reuse(FstMlaCtx* c, int32_t on) {
  if (!c) return fail(FST_MLA_ERR_ARG, "null context");
  c->plan_reuse = on != 0;
  return FST_MLA_OK;
}

int fst_cuda_mla_set_block_schedule(FstMlaCtx* c, int32_t on) {
  if (!c) return fail(FST_MLA_ERR_ARG, "null context");
  if (c->block_schedule != (on != 0)) c->planned = false;  // the next call builds its plan anew
  c->block_schedule = on != 0;
  return FST_MLA_OK;
}

int fst_cuda_mla_set_fused_merge(FstMlaCtx* c, int32_t on) {
  if (!c) return fail(FST_MLA_ERR_ARG, "null context");
  c->fused_merge = on != 0;
  return FST_MLA_OK;
}

int fst_cuda_mla_set_window(FstMlaCtx* c, int32_t window) {
  if (!c) return fail(FST_MLA_ERR_ARG, "null context");
  if (window < 0) return fail(FST_MLA_ERR_ARG, "negative window");
  c->window = window;
  return FST_MLA_OK;
}

int fst_cuda_mla_plan_counts(FstMlaCtx* c, int64_t* built, int64_t* reused) {
  if (!c) return fail(FST_MLA_ERR_ARG, "null context");
  if (built) *built = c->plans_built;
  if (reused) *reused = c->plans_reused;
  return FST_MLA_OK;
}

int fst_cuda_mla_plan_tokens(FstMlaCtx* c, int32_t* t_out) {
  if (!c || !t_out) return fail(FST_MLA_ERR_ARG, "null argument");
  if (!c->planned) return fail(FST_MLA_ERR_STATE, "no plan");
  *t_out = c->T;
  return FST_MLA_OK;
}

int fst_cuda_mla_plan_info(FstMlaCtx* c, int32_t* n_partials, int32_t* n_ctas, int64_t* kv_rows) {
  if (!c) return fail(FST_MLA_ERR_ARG, "null context");
  if (!c->planned) return fail(FST_MLA_ERR_STATE, "no plan");
  const Sched& S = c->sched[c->sched[c->info_class].built ? c->info_class : 0];
  if (n_partials) *n_partials = S.n_parts;
  if (n_ctas) *n_ctas = S.n_ctas;
  if (kv_rows) *kv_rows = S.kv_rows;
  return FST_MLA_OK;
}

/* ---- running -------------------------------------------------------------------------- */
int fst_cuda_mla_run_device(FstMlaCtx* c, int lid, const void* d_h_in, void* d_h_out) {
  int rc = check_run(c, lid);
  if (rc) return rc;
  if (!d_h_in || !d_h_out) return fail(FST_MLA_ERR_ARG, "null device pointer");
  if (c->T == 0) return FST_MLA_OK;
  CU(cudaSetDevice(c->cfg.device));
  if ((rc = prof_begin(c))) return rc;
  if ((rc = run_front(c, lid, (const bf16*)d_h_in))) return rc;
  prof_mark(c, FST_MLA_K_ATTN);
  bool direct = false;
  if ((rc = run_attention(c, lid, c->d_qeff, &direct))) return rc;
  prof_mark(c, FST_MLA_K_MERGE);
  if ((rc = run_merge_local(c, lid, 0, nullptr, direct))) return rc;
  if ((rc = run_back(c, lid, (bf16*)d_h_out))) return rc;
  c->cur = nullptr;
  CU(cudaGetLastError());
  return FST_MLA_OK;
}

int fst_cuda_mla_forward(FstMlaCtx* c, int lid, const uint16_t* h_in, uint16_t* h_out, const int32_t* seq_ids,
                         const int32_t* pos0, const int32_t* q_lens, int32_t n_seqs, int32_t causal) {
  if (!c || !h_in || !h_out || !seq_ids || !pos0 || !q_lens) return fail(FST_MLA_ERR_ARG, "null argument");
  if (n_seqs < 0) return fail(FST_MLA_ERR_ARG, "negative sequence count");
  std::vector<FstMlaSeqStep> steps(n_seqs);
  long long T_in = 0;
  for (int b = 0; b < n_seqs; ++b) {
    steps[b] = FstMlaSeqStep{seq_ids[b], pos0[b], q_lens[b], -1, 1, c->window};
    if (q_lens[b] > 0) T_in += q_lens[b];
  }
  // page-locked caller buffers are copied directly; pageable ones go through the context's
  // page-locked staging buffer (an asynchronous copy from pageable memory is neither)
  void* out_mapped = nullptr;  // the device's address of a page-locked, mapped h_out
  auto page_locked = [](const void* p, void** mapped) {
    cudaPointerAttributes at;
    if (cudaPointerGetAttributes(&at, p) != cudaSuccess) {
      cudaGetLastError();
      return false;
    }
    if (mapped && at.type == cudaMemoryTypeHost) *mapped = at.devicePointer;
    return at.type == cudaMemoryTypeHost;
  };
  // the input rows start their way to the device before the plan is built (the plan takes tens
  // of microseconds of host time and does not depend on them)
  const bool early = T_in > 0 && T_in <= c->cfg.max_tokens;
  const size_t bytes_in = (size_t)T_in * c->d.hidden * sizeof(uint16_t);
  const bool in_direct = page_locked(h_in, nullptr), out_direct = page_locked(h_out, &out_mapped);
  c->compress_done = false;
  // With a layer that can run, the plan is built in two parts: its per-token part goes to the
  // device at once, the front kernels start, and the split-KV schedule is built and uploaded on a
  // second stream while they run.
  const bool split = early && !c->profiling && lid >= 0 && lid < c->cfg.n_layers && c->layers[lid].set;
  if (early) {
    CU(cudaSetDevice(c->cfg.device));
    if (split) CU(cudaEventRecord(c->fwd_ev, c->stream));  // what was on the stream before this call
    if (!in_direct) memcpy(c->h_pinned, h_in, bytes_in);
    CU(cudaMemcpyAsync(c->d_h, in_direct ? (const void*)h_in : (const void*)c->h_pinned, bytes_in, cudaMemcpyHostToDevice, c->stream));
    // ... and so does the first GEMM of the layer (q / kv compression), which needs the rows and
    // the weights but nothing of the plan
    if (!c->profiling && lid >= 0 && lid < c->cfg.n_layers && c->layers[lid].set && !c->layers[lid].attn_norm) {
      int rc0 = run_gemm(c, plain_gemm(c->d_h, c->layers[lid].w_cmp, c->d_cmp, (int)T_in, c->d.cmp_n, c->d.hidden));
      if (rc0) return rc0;
      c->compress_done = true;
    }
  }
  bool reused = false;
  int rc = plan_tokens_part(c, steps.data(), n_seqs, causal, split, &reused);
  const bool two_parts = !rc && !reused && split && c->T > 0;
  if (!rc && !reused && !two_parts) rc = plan_schedule_part(c, false);
  if (rc) {
    c->compress_done = false;
    return rc;
  }
  if (!two_parts && (rc = check_run(c, lid))) return rc;
  if (c->T == 0) return FST_MLA_OK;
  const size_t bytes = (size_t)c->T * c->d.hidden * sizeof(uint16_t);
  // A page-locked output buffer that the device can address is written by the last GEMM itself
  // (512 KB of posted writes spread over the kernel) instead of by a copy behind it.
  const bool zero_copy = out_direct && out_mapped && c->out_zero_copy && !c->profiling;
  c->out_src = zero_copy ? (const bf16*)out_mapped : c->d_out;
  void* out_dev = zero_copy ? out_mapped : (void*)c->d_out;
  if (two_parts) {
    if ((rc = run_front(c, lid, c->d_h))) return rc;
    if ((rc = plan_schedule_part(c, true))) return rc;
    bool direct = false;
    if ((rc = run_attention(c, lid, c->d_qeff, &direct))) return rc;
    if ((rc = run_merge_local(c, lid, 0, nullptr, direct))) return rc;
    if ((rc = run_back(c, lid, (bf16*)out_dev))) return rc;
    CU(cudaGetLastError());
  } else if ((rc = fst_cuda_mla_run_device(c, lid, c->d_h, out_dev))) {
    return rc;
  }
  if (!zero_copy)
    CU(cudaMemcpyAsync(out_direct ? (void*)h_out : (void*)c->h_pinned, c->d_out, bytes, cudaMemcpyDeviceToHost, c->stream));
  // while the device works: the RoPE rows of the positions that a decode step asks for next
  for (int b = 0; b < n_seqs; ++b)
    if (q_lens[b] > 0 && q_lens[b] <= 4)
      for (int i = 0; i < q_lens[b]; ++i)
        for (int k = 0; k < 2; ++k)
          if (!c->lut_tag[k].empty()) lut_row_cached(c, k, pos0[b] + q_lens[b] + i);
  if ((rc = fst_cuda_mla_sync(c))) return rc;
  if (!out_direct) memcpy(h_out, c->h_pinned, bytes);
  return FST_MLA_OK;
}

int fst_cuda_mla_append_rows(FstMlaCtx* c, int lid, const uint16_t* h_in, const int32_t* seq_ids, const int32_t* pos0,
                             const int32_t* q_lens, int32_t n_seqs) {
  if (!c || !h_in || !seq_ids || !pos0 || !q_lens) return fail(FST_MLA_ERR_ARG, "null argument");
  if (n_seqs < 0) return fail(FST_MLA_ERR_ARG, "negative sequence count");
  std::vector<FstMlaSeqStep> steps(n_seqs);
  for (int b = 0; b < n_seqs; ++b) steps[b] = FstMlaSeqStep{seq_ids[b], pos0[b], q_lens[b], -1, 1, 0};
  int rc = fst_cuda_mla_plan(c, steps.data(), n_seqs, 0);
  if (rc) return rc;
  if ((rc = check_run(c, lid))) return rc;
  if (c->T == 0) return FST_MLA_OK;
  if (c->layers[lid].cmp_ratio) return fail(FST_MLA_ERR_STATE, "layer %d has a KV compressor: its rows come with a layer call", lid);
  CU(cudaSetDevice(c->cfg.device));
  const Dims& d = c->d;
  const LayerW& w = c->layers[lid];
  const size_t bytes = (size_t)c->T * d.hidden * sizeof(uint16_t);
  memcpy(c->h_pinned, h_in, bytes);
  CU(cudaMemcpyAsync(c->d_h, c->h_pinned, bytes, cudaMemcpyHostToDevice, c->stream));
  const bf16* rows = c->d_h;
  if (w.attn_norm) {
    launch_rmsnorm_rows(c->d_h, w.attn_norm, c->d_an, c->T, d.hidden, c->cfg.rms_eps, c->stream);
    c->launches += 1;
    rows = c->d_an;
  }
  if ((rc = run_gemm(c, plain_gemm(rows, w.w_cmp, c->d_cmp, c->T, d.cmp_n, d.hidden)))) return rc;
  NormAppendArgs na;
  na.cmp = c->d_cmp; na.q_norm = w.q_norm; na.kv_norm = w.kv_norm; na.lut = lut_of(c, lid);
  na.dst_row = c->d_dst; na.qc = c->d_qc; na.kv_new = c->d_kvnew; na.pool = c->pools[lid];
  na.T = c->T; na.q_lora = d.q_lora; na.kv_lora = d.kv_lora; na.row = d.row; na.rope = d.rope;
  na.eps = c->cfg.rms_eps;
  launch_norm_append(na, c->stream);
  c->launches += 1;
  CU(cudaGetLastError());
  return fst_cuda_mla_sync(c);
}

int fst_cuda_mla_attention_only(FstMlaCtx* c, int lid, const uint16_t* q_eff, uint16_t* o_lat) {
  int rc = check_run(c, lid);
  if (rc) return rc;
  if (!q_eff || !o_lat) return fail(FST_MLA_ERR_ARG, "null argument");
  if (c->T == 0) return FST_MLA_OK;
  CU(cudaSetDevice(c->cfg.device));
  const Dims& d = c->d;
  CU(cudaMemcpyAsync(c->d_qeff, q_eff, (size_t)c->T * d.H * d.d_qk * 2, cudaMemcpyHostToDevice, c->stream));
  if ((rc = prof_begin(c))) return rc;
  prof_mark(c, FST_MLA_K_ATTN);
  bool direct = false;
  if ((rc = run_attention(c, lid, c->d_qeff, &direct))) return rc;
  prof_mark(c, FST_MLA_K_MERGE);
  if ((rc = run_merge_local(c, lid, 0, nullptr, direct))) return rc;
  prof_mark(c, FST_MLA_K_OPROJ_A);
  c->cur = nullptr;
  CU(cudaMemcpyAsync(o_lat, c->d_olat, (size_t)c->T * d.H * d.d_v * 2, cudaMemcpyDeviceToHost, c->stream));
  return fst_cuda_mla_sync(c);
}

int fst_cuda_mla_run_partial_device(FstMlaCtx* c, int lid, const void* d_h_in, void* d_partial) {
  int rc = check_run(c, lid);
  if (rc) return rc;
  if (!d_h_in || !d_partial) return fail(FST_MLA_ERR_ARG, "null device pointer");
  if (c->T == 0) return FST_MLA_OK;
  CU(cudaSetDevice(c->cfg.device));
  if ((rc = prof_begin(c))) return rc;
  if ((rc = run_front(c, lid, (const bf16*)d_h_in))) return rc;
  prof_mark(c, FST_MLA_K_ATTN);
  if ((rc = run_attention(c, lid, c->d_qeff))) return rc;
  prof_mark(c, FST_MLA_K_MERGE);
  if ((rc = run_merge_local(c, lid, 1, (float*)d_partial))) return rc;
  prof_mark(c, FST_MLA_K_OPROJ_A);
  c->cur = nullptr;
  CU(cudaGetLastError());
  return FST_MLA_OK;
}

int fst_cuda_mla_run_merge_device(FstMlaCtx* c, int lid, const void* d_partials, int32_t n_parts, void* d_h_out) {
  int rc = check_run(c, lid);
  if (rc) return rc;
  if (!d_partials || !d_h_out || n_parts <= 0) return fail(FST_MLA_ERR_ARG, "bad partial buffer");
  if (c->T == 0) return FST_MLA_OK;
  CU(cudaSetDevice(c->cfg.device));
  const Dims& d = c->d;
  if ((rc = prof_begin(c))) return rc;
  prof_mark(c, FST_MLA_K_MERGE_GATHERED);
  MergeGatheredArgs m;
  m.parts = (const float*)d_partials; m.sinks = d.v4 ? c->layers[lid].sinks : nullptr; m.lut = lut_of(c, lid);
  m.o_lat = c->d_olat; m.n_parts = n_parts; m.T = c->T; m.H = d.H; m.d_v = d.d_v; m.rope = d.rope;
  m.inv_rope = inv_rope_heads(c, lid);
  launch_merge_gathered(m, c->stream);
  c->launches += 1;
  if ((rc = run_back(c, lid, (bf16*)d_h_out))) return rc;
  c->cur = nullptr;
  CU(cudaGetLastError());
  return FST_MLA_OK;
}

int fst_cuda_mla_get_stage(FstMlaCtx* c, int stage, uint16_t* host_out, size_t bytes) {
  if (!c || !host_out) return fail(FST_MLA_ERR_ARG, "null argument");
  if (!c->planned) return fail(FST_MLA_ERR_STATE, "no plan");
  const Dims& d = c->d;
  const bf16* src = nullptr;
  size_t n = 0;
  switch (stage) {
    case FST_MLA_STAGE_QC: src = c->d_qc; n = (size_t)c->T * d.q_lora; break;
    case FST_MLA_STAGE_KV: src = c->d_kvnew; n = (size_t)c->T * d.row; break;
    case FST_MLA_STAGE_QEFF: src = c->d_qeff; n = (size_t)c->T * d.H * d.d_qk; break;
    case FST_MLA_STAGE_OLAT: src = c->d_olat; n = (size_t)c->T * d.H * d.d_v; break;
    case FST_MLA_STAGE_LOW: src = c->d_low; n = (size_t)c->T * d.low; break;
    case FST_MLA_STAGE_OUT: src = c->out_src ? c->out_src : c->d_out; n = (size_t)c->T * d.hidden; break;
    default: return fail(FST_MLA_ERR_ARG, "unknown stage %d", stage);
  }
  if (bytes != n * 2) return fail(FST_MLA_ERR_ARG, "stage %d holds %zu bytes, caller asked for %zu", stage, n * 2, bytes);
  CU(cudaSetDevice(c->cfg.device));
  CU(cudaStreamSynchronize(c->stream));
  CU(cudaMemcpy(host_out, src, bytes, cudaMemcpyDefault));
  return FST_MLA_OK;
}

int fst_cuda_mla_gemm(FstMlaCtx* c, uint16_t* C, const uint16_t* A, const uint16_t* B, int M, int N, int K, int b_kn) {
  if (!c || !C || !A || !B) return fail(FST_MLA_ERR_ARG, "null argument");
  if (M <= 0 || N <= 0 || K <= 0) return fail(FST_MLA_ERR_ARG, "non-positive GEMM size");
  CU(cudaSetDevice(c->cfg.device));
  bf16 *dA = nullptr, *dB = nullptr, *dC = nullptr;
  int rc = dev_alloc(&dA, (size_t)M * K);
  if (!rc) rc = dev_alloc(&dB, (size_t)N * K);
  if (!rc) rc = dev_alloc(&dC, (size_t)M * N);
  cudaError_t e = cudaSuccess;
  if (!rc) {
    e = cudaMemcpyAsync(dA, A, (size_t)M * K * 2, cudaMemcpyHostToDevice, c->stream);
    if (e == cudaSuccess) e = cudaMemcpyAsync(dB, B, (size_t)N * K * 2, cudaMemcpyHostToDevice, c->stream);
    if (e == cudaSuccess) {
      GemmArgs g = plain_gemm(dA, dB, dC, M, N, K);
      if (b_kn) {
        g.b_kn = 1;
        g.ldb = N;
      }
      rc = run_gemm(c, g);
    }
    if (e == cudaSuccess && !rc) e = cudaMemcpyAsync(C, dC, (size_t)M * N * 2, cudaMemcpyDeviceToHost, c->stream);
    if (e == cudaSuccess && !rc) rc = fst_cuda_mla_sync(c);
  }
  cudaStreamSynchronize(c->stream);
  cudaFree(dA); cudaFree(dB); cudaFree(dC);
  if (e != cudaSuccess) return fail(FST_MLA_ERR_CUDA, "GEMM copy failed: %s", cudaGetErrorString(e));
  return rc;
}

/* ---- split-KV across GPUs: the exchange ------------------------------------------------- */
}  // extern "C"

namespace {

// NCCL through its C entry points, resolved at run time: the library already in the process (a
// host that uses NCCL itself has loaded it), else libnccl.so.2.
struct NcclApi {
  typedef struct { char internal[128]; } UniqueId;
  int (*GetUniqueId)(UniqueId*) = nullptr;
  int (*CommInitRank)(void**, int, UniqueId, int) = nullptr;
  int (*AllGather)(const void*, void*, size_t, int, void*, cudaStream_t) = nullptr;
  int (*CommDestroy)(void*) = nullptr;
  const char* (*GetErrorString)(int) = nullptr;
  bool ok = false;
};

NcclApi& nccl() {
  static NcclApi api;
  static bool tried = false;
  if (tried) return api;
  tried = true;
  void* h = dlopen("libnccl.so.2", RTLD_NOW | RTLD_NOLOAD);
  if (!h) h = dlopen("libnccl.so.2", RTLD_NOW | RTLD_GLOBAL);
  if (!h) h = dlopen("libnccl.so", RTLD_NOW | RTLD_GLOBAL);
  if (!h) return api;
  api.GetUniqueId = reinterpret_cast<decltype(api.GetUniqueId)>(dlsym(h, "ncclGetUniqueId"));
  api.CommInitRank = reinterpret_cast<decltype(api.CommInitRank)>(dlsym(h, "ncclCommInitRank"));
  api.AllGather = reinterpret_cast<decltype(api.AllGather)>(dlsym(h, "ncclAllGather"));
  api.CommDestroy = reinterpret_cast<decltype(api.CommDestroy)>(dlsym(h, "ncclCommDestroy"));
  api.GetErrorString = reinterpret_cast<decltype(api.GetErrorString)>(dlsym(h, "ncclGetErrorString"));
  api.ok = api.GetUniqueId && api.CommInitRank && api.AllGather && api.CommDestroy && api.GetErrorString;
  return api;
}

int comm_buffers(FstMlaCtx* c, int world) {
  const size_t rows = (size_t)c->cfg.max_tokens * c->d.H, w = 2 + (size_t)c->d.d_v;
  cudaFree(c->d_xpart);
  cudaFree(c->d_xgath);
  c->d_xpart = c->d_xgath = nullptr;
  int rc = dev_alloc(&c->d_xpart, rows * w);
  if (!rc) rc = dev_alloc(&c->d_xgath, rows * w * (size_t)world);
  return rc;
}

void comm_release(FstMlaCtx* c) {
  if (c->nccl_comm && nccl().ok) nccl().CommDestroy(c->nccl_comm);
  c->nccl_comm = nullptr;
  c->gather_fn = nullptr;
  c->gather_user = nullptr;
  cudaFree(c->d_xpart);
  cudaFree(c->d_xgath);
  c->d_xpart = c->d_xgath = nullptr;
  c->comm_world = 0;
}

}  // namespace

extern "C" {

int fst_cuda_mla_comm_unique_id(uint8_t id_out[128]) {
  if (!id_out) return fail(FST_MLA_ERR_ARG, "null argument");
  NcclApi& n = nccl();
  if (!n.ok) return fail(FST_MLA_ERR_COMM, "NCCL is not available (libnccl.so.2 could not be opened)");
  NcclApi::UniqueId id;
  const int r = n.GetUniqueId(&id);
  if (r != 0) return fail(FST_MLA_ERR_COMM, "ncclGetUniqueId: %s", n.GetErrorString(r));
  memcpy(id_out, id.internal, 128);
  return FST_MLA_OK;
}

int fst_cuda_mla_comm_init(FstMlaCtx* c, const uint8_t id[128], int32_t rank, int32_t world) {
  if (!c || !id) return fail(FST_MLA_ERR_ARG, "null argument");
  if (world < 1 || rank < 0 || rank >= world) return fail(FST_MLA_ERR_ARG, "rank %d of %d", rank, world);
  NcclApi& n = nccl();
  if (!n.ok) return fail(FST_MLA_ERR_COMM, "NCCL is not available (libnccl.so.2 could not be opened)");
  CU(cudaSetDevice(c->cfg.device));
  comm_release(c);
  NcclApi::UniqueId uid;
  memcpy(uid.internal, id, 128);
  void* comm = nullptr;
  const int r = n.CommInitRank(&comm, world, uid, rank);
  if (r != 0) return fail(FST_MLA_ERR_COMM, "ncclCommInitRank: %s", n.GetErrorString(r));
  c->nccl_comm = comm;
  c->comm_rank = rank;
  c->comm_world = world;
  return comm_buffers(c, world);
}

int fst_cuda_mla_comm_set_gather(FstMlaCtx* c, FstMlaGatherFn fn, void* user, int32_t rank, int32_t world) {
  if (!c || !fn) return fail(FST_MLA_ERR_ARG, "null argument");
  if (world < 1 || rank < 0 || rank >= world) return fail(FST_MLA_ERR_ARG, "rank %d of %d", rank, world);
  CU(cudaSetDevice(c->cfg.device));
  comm_release(c);
  c->gather_fn = fn;
  c->gather_user = user;
  c->comm_rank = rank;
  c->comm_world = world;
  return comm_buffers(c, world);
}

int fst_cuda_mla_comm_destroy(FstMlaCtx* c) {
  if (!c) return fail(FST_MLA_ERR_ARG, "null context");
  cudaSetDevice(c->cfg.device);
  cudaStreamSynchronize(c->stream);
  comm_release(c);
  return FST_MLA_OK;
}

int fst_cuda_mla_run_split_device(FstMlaCtx* c, int lid, const void* d_h_in, void* d_h_out) {
  int rc = check_run(c, lid);
  if (rc) return rc;
  if (!d_h_in || !d_h_out) return fail(FST_MLA_ERR_ARG, "null device pointer");
  if (c->comm_world < 1) return fail(FST_MLA_ERR_STATE, "no communicator: call fst_cuda_mla_comm_init first");
  if (c->T == 0) return FST_MLA_OK;
  CU(cudaSetDevice(c->cfg.device));
  const Dims& d = c->d;
  const size_t bytes = (size_t)c->T * d.H * (2 + d.d_v) * sizeof(float);
  if ((rc = prof_begin(c))) return rc;
  if ((rc = run_front(c, lid, (const bf16*)d_h_in))) return rc;
  prof_mark(c, FST_MLA_K_ATTN);
  if ((rc = run_attention(c, lid, c->d_qeff))) return rc;
  prof_mark(c, FST_MLA_K_MERGE);
  if ((rc = run_merge_local(c, lid, 1, c->d_xpart))) return rc;
  prof_mark(c, FST_MLA_K_EXCHANGE);
  if (c->gather_fn) {
    if (c->gather_fn(c->gather_user, c->d_xpart, c->d_xgath, bytes, c->stream) != 0)
      return fail(FST_MLA_ERR_COMM, "the host's gather function failed");
  } else {
    NcclApi& n = nccl();
    const int r = n.AllGather(c->d_xpart, c->d_xgath, bytes / sizeof(float), /* ncclFloat */ 7, c->nccl_comm, c->stream);
    if (r != 0) return fail(FST_MLA_ERR_COMM, "ncclAllGather: %s", n.GetErrorString(r));
  }
  prof_mark(c, FST_MLA_K_MERGE_GATHERED);
  MergeGatheredArgs m;
  m.parts = c->d_xgath; m.sinks = d.v4 ? c->layers[lid].sinks : nullptr; m.lut = lut_of(c, lid);
  m.o_lat = c->d_olat; m.n_parts = c->comm_world; m.T = c->T; m.H = d.H; m.d_v = d.d_v; m.rope = d.rope;
  m.inv_rope = inv_rope_heads(c, lid);
  launch_merge_gathered(m, c->stream);
  c->launches += 1;
  if ((rc = run_back(c, lid, (bf16*)d_h_out))) return rc;
  c->cur = nullptr;
  CU(cudaGetLastError());
  return FST_MLA_OK;
}

int fst_cuda_mla_forward_split(FstMlaCtx* c, int lid, const uint16_t* h_in, uint16_t* h_out,
                               const FstMlaSeqStep* steps, int32_t n_seqs, int32_t causal) {
  if (!c || !h_in || !h_out) return fail(FST_MLA_ERR_ARG, "null argument");
  int rc = fst_cuda_mla_plan(c, steps, n_seqs, causal);
  if (rc) return rc;
  if ((rc = check_run(c, lid))) return rc;
  if (c->T == 0) return FST_MLA_OK;
  CU(cudaSetDevice(c->cfg.device));
  const size_t bytes = (size_t)c->T * c->d.hidden * sizeof(uint16_t);
  memcpy(c->h_pinned, h_in, bytes);
  CU(cudaMemcpyAsync(c->d_h, c->h_pinned, bytes, cudaMemcpyHostToDevice, c->stream));
  c->out_src = c->d_out;
  if ((rc = fst_cuda_mla_run_split_device(c, lid, c->d_h, c->d_out))) return rc;
  CU(cudaMemcpyAsync(c->h_pinned, c->d_out, bytes, cudaMemcpyDeviceToHost, c->stream));
  if ((rc = fst_cuda_mla_sync(c))) return rc;
  memcpy(h_out, c->h_pinned, bytes);
  return FST_MLA_OK;
}

/* ---- measurement ---------------------------------------------------------------------- */
int fst_cuda_mla_launch_count(FstMlaCtx* c, int64_t* n_out) {
  if (!c || !n_out) return fail(FST_MLA_ERR_ARG, "null argument");
  *n_out = c->launches;
  return FST_MLA_OK;
}

int fst_cuda_mla_family_counts(FstMlaCtx* c, int64_t* tensor_out, int64_t* simt_out) {
  if (!c) return fail(FST_MLA_ERR_ARG, "null context");
  if (tensor_out) *tensor_out = c->launches_tensor;
  if (simt_out) *simt_out = c->launches_simt;
  return FST_MLA_OK;
}

int fst_cuda_mla_selftest_wait_expiry(FstMlaCtx* c, int32_t polls) {
  if (!c) return fail(FST_MLA_ERR_ARG, "null context");
  if (polls < 1 || polls > (1 << 16)) return fail(FST_MLA_ERR_ARG, "poll limit %d outside [1, 65536]", polls);
  CU(cudaSetDevice(c->cfg.device));
  c->status_by_kernel = false;
  launch_wait_selftest(c->d_status, (uint32_t)polls, c->stream);
  c->launches += 1;
  CU(cudaGetLastError());
  return FST_MLA_OK;
}

int fst_cuda_mla_debug_attr_first_use(uint64_t kernel_key, int32_t device, int64_t value) {
  return kernel_attr_registry().first_use(reinterpret_cast<const void*>(static_cast<uintptr_t>(kernel_key)), device,
                                          value) ? 1 : 0;
}

int fst_cuda_mla_debug_schedule(int32_t n_sm, const int32_t* pos0, const int32_t* q_lens, int32_t n_seqs, int32_t causal,
                                int32_t by_blocks, int32_t* segs_out, int32_t cap, int32_t* n_segs_out, int32_t* n_ctas_out,
                                int32_t* cut_by_blocks_out) {
  if (!pos0 || !q_lens || !segs_out || !n_segs_out || !n_ctas_out || n_sm < 1 || n_seqs < 0 || cap < 0)
    return fail(FST_MLA_ERR_ARG, "bad argument");
  // a context that never touches a device: only what the two cutting functions read
  FstMlaCtx c;
  memset(&c.cfg, 0, sizeof(c.cfg));
  c.cfg.page_tokens = 64;
  c.n_sm = n_sm;
  c.pl_causal = causal;
  int T = 0;
  for (int b = 0; b < n_seqs; ++b) {
    if (pos0[b] < 0 || q_lens[b] < 0) return fail(FST_MLA_ERR_ARG, "negative position or length");
    c.pl_steps.push_back(FstMlaSeqStep{b, pos0[b], q_lens[b], -1, 1, 0});
    for (int i = 0; i < q_lens[b]; ++i, ++T) {
      c.pl_tok_table.push_back(b);  // stands for the offset of the sequence's block table
      c.pl_kvlen.push_back(causal ? pos0[b] + i + 1 : pos0[b] + q_lens[b]);
      c.pl_kvlo.push_back(0);
    }
  }
  std::vector<AttnSeg> segs;
  std::vector<int32_t> cta_seg, tok_part;
  long long kv_rows = 0;
  bool blocks = by_blocks && cut_block_schedule(&c, T, &segs, &cta_seg, &tok_part, &kv_rows);
  if (!blocks) {
    std::vector<TileStream> streams;
    for (int t = 0; t < T; ++t) streams.push_back(TileStream{t, c.pl_tok_table[t], 0, c.pl_kvlen[t]});
    cut_schedule(&c, streams, T, &segs, &cta_seg, &tok_part, &kv_rows);
  }
  if ((int)segs.size() > cap) return fail(FST_MLA_ERR_CAPACITY, "%d segments, room for %d", (int)segs.size(), cap);
  const int n_ctas = (int)cta_seg.size() - 1;
  for (int k = 0; k < n_ctas; ++k)
    for (int i = cta_seg[k]; i < cta_seg[k + 1]; ++i) {
      int32_t* o = segs_out + 5 * (size_t)i;
      o[0] = segs[i].tok; o[1] = segs[i].kv_begin; o[2] = segs[i].kv_end; o[3] = segs[i].part; o[4] = k;
      if (segs[i].part < tok_part[segs[i].tok] || segs[i].part >= tok_part[segs[i].tok + 1])
        return fail(FST_MLA_ERR_STATE, "segment %d: part %d outside its token's range", i, segs[i].part);
    }
  *n_segs_out = (int)segs.size();
  *n_ctas_out = n_ctas;
  if (cut_by_blocks_out) *cut_by_blocks_out = blocks ? 1 : 0;
  return FST_MLA_OK;
}

int fst_cuda_mla_debug_set_status(FstMlaCtx* c, int32_t code) {
  if (!c) return fail(FST_MLA_ERR_ARG, "null context");
  c->status_by_kernel = false;
  CU(cudaSetDevice(c->cfg.device));
  CU(cudaMemcpyAsync(c->d_status, &code, sizeof(int), cudaMemcpyHostToDevice, c->stream));
  CU(cudaStreamSynchronize(c->stream));
  return FST_MLA_OK;
}

int fst_cuda_mla_set_profiling(FstMlaCtx* c, int on) {
  if (!c) return fail(FST_MLA_ERR_ARG, "null context");
  c->profiling = on != 0;
  return FST_MLA_OK;
}

int fst_cuda_mla_kernel_times(FstMlaCtx* c, float* ms_out, int32_t* n_out) {
  if (!c || !ms_out || !n_out) return fail(FST_MLA_ERR_ARG, "null argument");
  CU(cudaSetDevice(c->cfg.device));
  int rc = prof_flush(c);
  if (rc) return rc;
  for (int k = 0; k < FST_MLA_K_COUNT; ++k) {
    ms_out[k] = c->k_ms[k];
    n_out[k] = c->k_n[k];
    c->k_ms[k] = 0;
    c->k_n[k] = 0;
  }
  return FST_MLA_OK;
}

}  // extern "C"
