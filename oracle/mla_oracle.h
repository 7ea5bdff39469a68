/* CPU oracle for the FaStar MLA layer.  TEST INFRASTRUCTURE ONLY.
 *
 * A plain C++ restatement of the arithmetic of FSTEngine::process_mla
 * (reference src/fst_engine.cpp:3320-3890) and of the helpers it calls.  It is
 * the checker the CUDA path is compared against and the host-CPU baseline the
 * benchmark times; nothing in the shipped library links or calls it.
 *
 * Parity status: the elementary pieces (RMSNorm, RoPE tables, sink softmax,
 * latent attention, bf16 helpers) are pinned against outputs of the reference's
 * own functions (tests/golden/).  The reference holds no stored end-to-end
 * vectors for process_mla and its GEMMs only run on an XDNA2 NPU, so the full
 * layer composition is pinned by formula, not by stored values.
 *
 * All tensors are float arrays holding either fp32 values (round_bf16 == 0) or
 * bf16-representable values (round_bf16 == 1: every stage boundary is rounded
 * to bf16, round-to-nearest-even, where the reference stores a bf16 buffer).
 * Weight matrices are [N_out, K_in] row-major, consumed as C = A * B^T
 * (reference src/fst_engine.cpp:1611-1615).
 */
#ifndef FST_MLA_ORACLE_H
#define FST_MLA_ORACLE_H
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

enum { FST_ORACLE_PRESET_BASELINE = 0, FST_ORACLE_PRESET_FASTAR_V4 = 1 };

typedef struct {
  int32_t preset;        /* FST_ORACLE_PRESET_* */
  int32_t hidden;        /* 4096 */
  int32_t n_heads;       /* 64 */
  int32_t q_lora;        /* 1024 */
  int32_t kv_lora;       /* 512 */
  int32_t qk_nope;       /* BASELINE: 128.  V4: head_dim - qk_rope = 448 */
  int32_t qk_rope;       /* 64 */
  int32_t v_head;        /* BASELINE: 128.  V4: unused */
  int32_t o_groups;      /* V4: 8 groups of wo_a.  BASELINE: unused */
  int32_t o_lora;        /* V4: 1024 rows of wo_a per group */
  float softmax_scale;   /* BASELINE 1/sqrt(192); V4 1/sqrt(512) */
  float rope_theta;      /* 10000 */
  float rms_eps;         /* 1e-6 */
  int32_t rope_yarn;     /* 0: plain; 1: YaRN tables of compressed V4 layers */
  int32_t use_sink;      /* V4: per-head sink logit in the softmax denominator */
  int32_t round_bf16;    /* 1: round every stage boundary to bf16 */
  int32_t n_threads;     /* worker threads (<=0: one per available core) */
  int32_t draft_form;    /* V4: the draft model's layer (process_draft_mla, src/fst_engine.cpp:4884-5131):
                            no per-head q norm, q and inverse output rotation on head 0 only */
  int32_t window;        /* > 0: a query row attends only to the last `window` raw rows it may see (the
                            draft model keeps window_size rows in a ring, 2534-2576); whole-layer calls only */
} FstOracleCfg;

/* Weights for one layer.  Unused members may be NULL.
 * BASELINE: wq_a[q_lora,hidden] wq_b[H*(nope+rope),q_lora] wkv_a[kv_lora+rope,hidden]
 *           wkv_b[H*(nope+v_head),kv_lora] (per head: nope rows W_UK then v_head rows W_UV)
 *           wo_b[hidden,H*v_head] q_norm[q_lora] kv_norm[kv_lora]
 * V4:       wq_a[q_lora,hidden] wq_b[H*512,q_lora] wkv_a[512,hidden]
 *           wo_a[o_groups*o_lora, H*512/o_groups] wo_b[hidden,o_groups*o_lora]
 *           q_norm kv_norm attn_sinks[H]
 * attn_norm[hidden] (either preset, may be NULL): the weighted RMSNorm that process_layer applies
 * to the rows before it calls process_mla (reference src/fst_engine.cpp:2687-2689); when set,
 * `h` holds the rows before that norm. */
typedef struct {
  const float* wq_a;
  const float* wq_b;
  const float* wkv_a;
  const float* wkv_b;
  const float* wo_a;
  const float* wo_b;
  const float* q_norm;
  const float* kv_norm;
  const float* attn_sinks;
  const float* attn_norm;
} FstOracleWeights;

/* Optional per-stage dumps (the FST_MLA_TRACE stage list, reference
 * src/fst_engine.cpp:3330-3340, 3396-3407, 3521-3532, 3685-3695, 3841-3851).
 * Any pointer may be NULL. Sizes for M new tokens:
 * qc[M,q_lora] kv[M,row] q_eff[M*H,d_qk] o_lat[M*H,d_v] low[M,low_dim] */
typedef struct {
  float* qc;
  float* kv;
  float* q_eff;
  float* o_lat;
  float* low;
} FstOracleTrace;

int fst_oracle_row_width(const FstOracleCfg* c);  /* cache row: 576 (BASELINE) / 512 (V4) */
int fst_oracle_d_qk(const FstOracleCfg* c);
int fst_oracle_d_v(const FstOracleCfg* c);
int fst_oracle_low_dim(const FstOracleCfg* c);    /* 8192 for both presets */
int fst_oracle_threads(const FstOracleCfg* c);    /* threads a call will use */

/* bf16 helpers. round: RNE (this build).  trunc: the reference's f2bf
 * (src/fst_engine.cpp:27). */
float fst_oracle_bf16_round(float x);
float fst_oracle_bf16_trunc(float x);
void fst_oracle_bf16_round_array(float* x, int64_t n);

/* y = x * w / sqrt(mean(x^2) + eps), rows x d.  w may be NULL (weightless).
 * Follows rms_cpu, reference src/fst_engine.cpp:89-91. */
void fst_oracle_rmsnorm(const float* x, const float* w, float* y, int rows, int d, float eps,
                        int round_bf16);

/* cos/sin table for rope_dim/2 pairs at position pos: lut[2j]=cos, lut[2j+1]=sign*sin.
 * Follows build_rope_lut, reference src/fst_engine.cpp:1970-2023 (the angle of pair j is
 * obtained by repeated multiplication by theta_scale, as there). round_lut_bf16 reproduces the
 * reference's bf16 table entries. */
void fst_oracle_rope_lut(float* lut, int pos, int rope_dim, float theta, int yarn, int inverse,
                         int round_lut_bf16);

/* Interleaved-pair rotation of x[rope_dim] in place at position pos
 * (ew_rope, reference kernels/fst_ew_unified_kernel.cc:200-217). */
void fst_oracle_rope_apply(float* x, int pos, int rope_dim, float theta, int yarn, int inverse,
                           int round_bf16);

/* C[M,N] = A[M,K] * B[N,K]^T (b_kn == 0) or A[M,K] * B[K,N] (b_kn == 1). */
void fst_oracle_gemm(const float* A, const float* B, float* C, int M, int N, int K, int b_kn,
                     int round_bf16, int n_threads);

/* Latent attention of one sequence (reference src/fst_engine.cpp:3573-3683).
 * q_eff[n_q*H, d_qk]; cache[L, row] with keys = row[:d_qk], values = row[:d_v].
 * Query token i attends to cache rows s < kv_len and, if causal, s <= pos0 + i.
 * sinks: NULL or [H].  out[n_q*H, d_v]. */
void fst_oracle_attention(const FstOracleCfg* c, const float* q_eff, const float* cache,
                          int kv_len, int n_q, int pos0, int causal, const float* sinks,
                          float* out);

/* Split-KV form of the same attention over cache rows [s0, s1): un-normalised partials
 * m[n_q*H], l[n_q*H], o[n_q*H, d_v] with l = sum exp(s - m), o = sum exp(s - m) * v.
 * P is not rounded here. */
void fst_oracle_attention_partial(const FstOracleCfg* c, const float* q_eff, const float* cache,
                                  int s0, int s1, int n_q, int pos0, int causal, float* m,
                                  float* l, float* o);

/* Log-sum-exp merge of n_parts partials laid out [part][rows] / [part][rows, d_v];
 * sinks NULL or [H] (row r uses head r % H). out[rows, d_v] normalised. */
void fst_oracle_merge_partials(const FstOracleCfg* c, const float* m, const float* l,
                               const float* o, int n_parts, int rows, const float* sinks,
                               float* out);

/* The whole layer for one sequence: M new tokens h[M,hidden] at positions
 * pos0 .. pos0+M-1.  cache[cap, row] holds rows [0,pos0) on entry and rows
 * [0,pos0+M) on return (append, reference src/fst_engine.cpp:3534-3544).
 * out[M,hidden].  Returns 0, or -1 when pos0 + M > cap (the reference asserts). */
int fst_oracle_mla_forward(const FstOracleCfg* c, const FstOracleWeights* w, const float* h, int M,
                           int pos0, int causal, float* cache, int cap, float* out,
                           FstOracleTrace* trace);

/* ---- V4 KV compressor (reference src/fst_engine.cpp:3063-3318) ---------------------------------
 * Layers whose compress ratio is 4 or 128 stream every token's attn-normed hidden row through a
 * per-layer compressor: two projections (wkv, wgate: [width, hidden], width = 1024 for ratio 4, 512
 * for ratio 128), a positional bias (ape [ratio, width]) on the gate, a window state, and on every
 * ratio-th token one pooled, normed (norm [kv_lora]), tail-rotated, E4M3-round-tripped row of
 * kv_lora values that joins the attention as one more column (3565-3586, 3630-3635). */
typedef struct {
  int32_t ratio;       /* 4 or 128 (0: no compressor) */
  const float* wkv;    /* [width, hidden] */
  const float* wgate;  /* [width, hidden] */
  const float* ape;    /* [ratio, width] */
  const float* norm;   /* [kv_lora] */
} FstOracleCompressorW;

/* Streaming state of one (layer, sequence): state_kv / state_sc are [rows, width] with rows = 8 for
 * ratio 4 (two lanes of four) and `ratio` otherwise; the engine starts them at zero
 * (reset_compressor_state, 3160-3169).  cache[cap, kv_lora] receives the compressed rows. */
typedef struct {
  float* state_kv;
  float* state_sc;
  float* cache;
  int32_t n_comp;
  int32_t cap;
} FstOracleCompressorState;

int fst_oracle_compressor_width(int ratio, int kv_lora);
int fst_oracle_compressor_rows(int ratio);
/* e4m3_roundtrip (3084-3100): nearest of the 127 non-negative E4M3 values, the reference's tie rule. */
float fst_oracle_e4m3_roundtrip(float v);
/* compress_token (3171-3318) for the token at position `pos` (the sequence's positions must arrive
 * in order from 0).  Returns 1 when a row was emitted, 0 when not, -1 when the cache is full. */
int fst_oracle_compress_token(const FstOracleCfg* c, const FstOracleCompressorW* w, FstOracleCompressorState* st,
                              const float* hidden_normed, int pos);

/* The same layer for B sequences in one call (batched decode): h[T, hidden] holds the rows of
 * the sequences back to back (T = sum q_lens), caches[b] is sequence b's [caps[b], row] buffer.
 * Every row gets exactly the arithmetic of fst_oracle_mla_forward; the projections run over all
 * T rows at once so the weights are read once per call.  Trace buffers hold T rows. */
int fst_oracle_mla_forward_batch(const FstOracleCfg* c, const FstOracleWeights* w, const float* h, int B,
                                 const int32_t* q_lens, const int32_t* pos0, int causal, float* const* caches,
                                 const int32_t* caps, float* out, FstOracleTrace* trace);
/* ... with the layer's KV compressor: cw (ratio 4 or 128) and one state per sequence.  The new rows
 * go through the compressor after the cache push and before the attention (3545-3568), and every
 * query row attends to its raw rows AND to the compressed rows it may see: all of them in decode,
 * those emitted at a position <= its own when causal (3630-3635). */
int fst_oracle_mla_forward_batch_cmp(const FstOracleCfg* c, const FstOracleWeights* w,
                                     const FstOracleCompressorW* cw, FstOracleCompressorState* states,
                                     const float* h, int B, const int32_t* q_lens, const int32_t* pos0, int causal,
                                     float* const* caches, const int32_t* caps, float* out, FstOracleTrace* trace);

/* Host twin of the paged-cache bookkeeping: a LIFO free list of n_pages pages.
 * Used to check page mapping bit-exactly.  Opaque handle. */
typedef struct FstOraclePager FstOraclePager;
FstOraclePager* fst_oracle_pager_create(int n_pages, int page_tokens, int max_seqs);
void fst_oracle_pager_destroy(FstOraclePager* p);
int fst_oracle_pager_seq_alloc(FstOraclePager* p);                 /* seq id or -1 */
int fst_oracle_pager_seq_free(FstOraclePager* p, int seq);
int fst_oracle_pager_reserve(FstOraclePager* p, int seq, int n_tokens); /* grow to n tokens */
int fst_oracle_pager_truncate(FstOraclePager* p, int seq, int n_tokens);
int fst_oracle_pager_table(const FstOraclePager* p, int seq, int32_t* out, int cap);
int fst_oracle_pager_free_pages(const FstOraclePager* p);

#ifdef __cplusplus
}
#endif
#endif
