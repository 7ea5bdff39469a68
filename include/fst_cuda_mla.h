/* C ABI of the B200 (sm_100a) Multi-head Latent Attention path of the FaStar engine.
 *
 * This is the boundary FSTEngine::process_mla (reference src/fst_engine.cpp:3320-3890,
 * declared include/fst_engine.h:309) crosses instead of the NPU dispatch helpers
 * (npu_gemm_mla_vec 465-575, npu_rmsnorm_weighted 882-934, npu_rope 815-856) and the XRT
 * buffer objects bo_mla_* / KVCacheEntry (include/fst_engine.h:108-113, 533-557).
 *
 * Plain C: pointers and sizes only.  Every function returns FST_MLA_OK (0) or a negative
 * FST_MLA_ERR_* code and never throws; fst_cuda_mla_last_error() describes the last
 * failure of the calling thread.  The engine's wrapper turns a non-zero code into the
 * std::runtime_error the reference raises (src/fst_engine.cpp:200-223).
 *
 * Threading: one context per GPU, calls serialised by the caller (the reference is single
 * threaded, src/fst_main.cpp:461,506).  All work of a context runs on one CUDA stream.
 *
 * bf16 values cross the boundary as uint16_t bit patterns (bf16_t of include/fst_engine.h:16).
 * Weight matrices are [N_out, K_in] row-major, consumed as C = A * B^T, exactly as the
 * reference holds them (src/fst_engine.cpp:1611-1615).
 */
#ifndef FST_CUDA_MLA_H
#define FST_CUDA_MLA_H
#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define FST_MLA_OK 0
#define FST_MLA_ERR_ARG (-1)          /* bad argument */
#define FST_MLA_ERR_PAGES (-2)        /* the page pool is exhausted */
#define FST_MLA_ERR_CAPACITY (-3)     /* too many sequences / tokens for this context */
#define FST_MLA_ERR_CUDA (-4)         /* a CUDA call failed */
#define FST_MLA_ERR_DEVICE_CHECK (-5) /* a kernel gave up a bounded wait or failed a check */
#define FST_MLA_ERR_STATE (-6)        /* call order: no weights, no plan */
#define FST_MLA_ERR_NO_DEVICE (-7)    /* no CUDA device: there is no CPU fallback */
#define FST_MLA_ERR_COMM (-8)         /* the exchange between GPUs failed (NCCL missing or a call of it) */

#define FST_MLA_PRESET_BASELINE 0  /* 576-wide rows [512 latent | 64 k_pe], W_UK absorb, per-head W_UV */
#define FST_MLA_PRESET_FASTAR_V4 1 /* live engine: 512-wide rows, RoPE tail, sink, grouped wo_a */

/* Kernel selection (for bisecting; AUTO is what the engine uses). */
#define FST_MLA_IMPL_AUTO 0
#define FST_MLA_IMPL_TENSOR 1 /* tcgen05 / TMEM / TMA kernels */
#define FST_MLA_IMPL_SIMT 2   /* CUDA-core kernels (any shape) */

typedef struct FstMlaCtx FstMlaCtx;

/* Shape constants mirror include/fst_engine.h:92-95 (MLA_Q_LORA, MLA_KV_LORA, MLA_N_HEADS,
 * MLA_HEAD_DIM, MLA_ROPE_DIM) and ModelConfig (127-139). */
typedef struct FstMlaConfig {
  int32_t preset;
  int32_t hidden;    /* 4096 */
  int32_t n_heads;   /* 64 */
  int32_t q_lora;    /* 1024 */
  int32_t kv_lora;   /* 512 */
  int32_t qk_nope;   /* BASELINE 128 (V4: ignored, kv_lora - qk_rope) */
  int32_t qk_rope;   /* 64 */
  int32_t v_head;    /* BASELINE 128 */
  int32_t o_groups;  /* V4: 8 */
  int32_t o_lora;    /* V4: 1024 */
  float softmax_scale; /* <= 0: preset default (1/sqrt(nope+rope) or 1/sqrt(kv_lora)) */
  float rope_theta;    /* 10000 */
  float rms_eps;       /* 1e-6 */
  int32_t rope_yarn;   /* RoPE kind every layer starts with: 0 plain, 1 the YaRN tables of the V4
                          compressed layers (src/fst_engine.cpp:1995-2022); per layer:
                          fst_cuda_mla_set_layer_rope */
  int32_t n_layers;
  int32_t page_tokens; /* 64 */
  int32_t n_pages;     /* pages per layer in the pool */
  int32_t max_seqs;
  int32_t max_tokens;  /* most new tokens (sum of q_len) in one call */
  int32_t device;      /* CUDA ordinal */
  int32_t attn_impl;   /* FST_MLA_IMPL_* */
  int32_t gemm_impl;   /* FST_MLA_IMPL_* */
} FstMlaConfig;

/* Host pointers, copied to the device once (replaces preload_all_layers,
 * src/fst_engine.cpp:1152-1197).  Members a preset does not use may be NULL.
 * BASELINE: wq_a[q_lora,hidden] wq_b[H*(nope+rope),q_lora] wkv_a[kv_lora+rope,hidden]
 *           wkv_b[H*(nope+v_head),kv_lora] (per head: W_UK rows then W_UV rows)
 *           wo_b[hidden,H*v_head] q_norm[q_lora] kv_norm[kv_lora]
 * V4 (LayerWeightsC, include/fst_engine.h:165-188): wq_a wq_b[H*512,q_lora] wkv_a = wkv[512,hidden]
 *           wo_a[o_groups*o_lora, H*512/o_groups] wo_b[hidden,o_groups*o_lora]
 *           q_norm kv_norm attn_sinks[H] (NULL: sink logit 0, src/fst_engine.cpp:3623)
 * attn_norm[hidden] (either preset, may be NULL): the weight of the RMSNorm that process_layer
 * applies in front of process_mla (src/fst_engine.cpp:2687-2689).  When it is set the layer call
 * takes the rows BEFORE that norm and applies it on the device. */
typedef struct FstMlaWeights {
  const uint16_t* wq_a;
  const uint16_t* wq_b;
  const uint16_t* wkv_a;
  const uint16_t* wkv_b;
  const uint16_t* wo_a;
  const uint16_t* wo_b;
  const uint16_t* q_norm;
  const uint16_t* kv_norm;
  const float* attn_sinks;
  const uint16_t* attn_norm;
} FstMlaWeights;

/* One sequence's share of a layer call.  The reference passes this implicitly as
 * seq_pos_ / M / is_prefill_ (src/fst_engine.cpp:3327, 3345, 3626). */
typedef struct FstMlaSeqStep {
  int32_t seq;       /* id from fst_cuda_mla_seq_alloc */
  int32_t pos0;      /* cache row of the first new token (seq_pos_) */
  int32_t q_len;     /* new tokens (M) */
  int32_t rope_pos0; /* RoPE position of the first new token; < 0: same as pos0 */
  int32_t append;    /* 1: write the new rows and attend to [0, pos0+q_len);
                        0: attend to [0, pos0) only (a KV slice that does not own them) */
  int32_t window;    /* > 0: every new token attends only to the last `window` rows it may see
                        (the draft model's sliding window, src/fst_engine.cpp:2534-2576 keeps
                        window_size rows in a ring); <= 0: to all of them */
} FstMlaSeqStep;

/* Intermediate buffers of the last run, the stage list of FST_MLA_TRACE
 * (src/fst_engine.cpp:3396-3407, 3521-3532, 3685-3695, 3841-3851). */
#define FST_MLA_STAGE_QC 0    /* [T, q_lora]      after wq_a + q_norm */
#define FST_MLA_STAGE_KV 1    /* [T, row]         new cache rows (normed latent, rotated k_pe) */
#define FST_MLA_STAGE_QEFF 2  /* [T*H, d_qk]      query in latent space, RoPE applied */
#define FST_MLA_STAGE_OLAT 3  /* [T*H, d_v]       attention output (V4: after inverse RoPE) */
#define FST_MLA_STAGE_LOW 4   /* [T, 8192]        after O-proj a */
#define FST_MLA_STAGE_OUT 5   /* [T, hidden]      after O-proj b */

/* Kernels whose device time fst_cuda_mla_kernel_times reports, in launch order. */
#define FST_MLA_K_COMPRESS 0 /* h * [wq_a; wkv_a]^T */
#define FST_MLA_K_NORM_APPEND 1
#define FST_MLA_K_Q_EXPAND 2
#define FST_MLA_K_Q_ABSORB 3 /* RoPE(q_pe) + W_UK absorb (V4: head RMSNorm + RoPE) */
#define FST_MLA_K_ATTN 4     /* split-KV QK / online softmax / SV over the paged cache */
#define FST_MLA_K_MERGE 5    /* log-sum-exp merge of the split partials */
#define FST_MLA_K_EXCHANGE 6 /* split-KV across GPUs: the all-gather of the per-GPU partials */
#define FST_MLA_K_MERGE_GATHERED 7 /* ... and the merge of the gathered partials */
#define FST_MLA_K_OPROJ_A 8
#define FST_MLA_K_OPROJ_B 9
#define FST_MLA_K_COUNT 10

/* ---- lifetime ------------------------------------------------------------------------- */
/* Replaces device probe + buffer allocation of FSTEngine::FSTEngine (src/fst_engine.cpp:
 * 1250-1270, 1419-1474).  Fails with FST_MLA_ERR_NO_DEVICE when there is no GPU. */
int fst_cuda_mla_create(const FstMlaConfig* cfg, FstMlaCtx** out);
void fst_cuda_mla_destroy(FstMlaCtx* ctx);
const char* fst_cuda_mla_last_error(void);
/* Stream all later work is enqueued on (a cudaStream_t; NULL = the default stream). */
int fst_cuda_mla_set_stream(FstMlaCtx* ctx, void* cuda_stream);
/* Blocks until the stream is idle; reports a pending device-side check (npu_run_wait /
 * flush_pending_runs, src/fst_engine.cpp:200-223). */
int fst_cuda_mla_sync(FstMlaCtx* ctx);

/* ---- weights -------------------------------------------------------------------------- */
int fst_cuda_mla_set_layer_weights(FstMlaCtx* ctx, int lid, const FstMlaWeights* w);

/* RoPE kind of one layer.  build_rope_lut (src/fst_engine.cpp:1970-2023) chooses per layer: plain
 * RoPE with the model's base for layers whose compress ratio is 0, YaRN (base 160000, scale 1/16)
 * for the others (1979-1982).  yarn: 0 plain, 1 YaRN.  q, k and the V4 inverse output rotation of
 * that layer all use the chosen table; a context whose layers differ keeps both tables per plan. */
int fst_cuda_mla_set_layer_rope(FstMlaCtx* ctx, int lid, int32_t yarn);
/* Base of the plain RoPE tables (FstMlaConfig.rope_theta) when it is only known after the
 * context exists: the engine takes it from the checkpoint header (rope_freq_base_,
 * src/fst_engine.cpp:1505). */
int fst_cuda_mla_set_rope_theta(FstMlaCtx* ctx, float theta);

/* The draft model's form of the layer (process_draft_mla, src/fst_engine.cpp:4884-5131; V4 form
 * only): no per-head query RMSNorm, the query's tail rotation and the inverse rotation of the
 * output on head 0 only (4967-4983, 5077-5093), dense attention over the rows that are there.  The
 * rest -- projections, norms, key RoPE by cache index, sink softmax, grouped wo_a, wo_b -- is the
 * main layer's.  The host drives it as process_draft_mla does: the projected main hidden row is
 * appended at the anchor position (fst_cuda_mla_append_rows), the candidate block is a
 * non-causal layer call at anchor + 1 whose rows are dropped again afterwards
 * (fst_cuda_mla_seq_truncate), and FstMlaSeqStep.window keeps the attention on the last
 * window_size main rows plus the block. */
int fst_cuda_mla_set_layer_draft_form(FstMlaCtx* ctx, int lid, int32_t on);
/* KV side of the layer alone: h rows -> kv compress, kv_norm, key RoPE, cache append; no attention
 * (the draft model's "main_kv from main_x", 4913-4940).  Host bf16 rows [sum q_lens, hidden]. */
int fst_cuda_mla_append_rows(FstMlaCtx* ctx, int lid, const uint16_t* h_in, const int32_t* seq_ids,
                             const int32_t* pos0, const int32_t* q_lens, int32_t n_seqs);

/* V4 KV compressor of one layer (reference LayerWeightsC cmp_*, include/fst_engine.h:172-180,
 * loaded at src/fst_engine.cpp:1657-1690; compress_token 3171-3318).  Layers whose compress ratio
 * is 4 or 128 stream every row through the compressor in front of the attention (3545-3568): every
 * ratio-th row emits one pooled, normed, tail-rotated, E4M3-round-tripped row of kv_lora values, and
 * those rows are further attention columns (3565-3586) with the causal rule of 3630-3635.  Here they
 * live in pages of their own (a second block table per sequence); the window state is kept per
 * (layer, sequence) on the device.  width = 2 * kv_lora for ratio 4, kv_lora for ratio 128.
 * Host pointers, copied once.  V4 form only.  Set before any sequence holds rows; w == NULL or
 * ratio 0 removes the compressor.  A sequence's rows must then reach the layer in order from row 0
 * (fst_cuda_mla_cache_write does not go through the compressor). */
typedef struct FstMlaCompressor {
  int32_t ratio;         /* 4 or 128 */
  const uint16_t* wkv;   /* bf16 [width, hidden] */
  const uint16_t* wgate; /* bf16 [width, hidden] */
  const float* ape;      /* fp32 [ratio, width] */
  const uint16_t* norm;  /* bf16 [kv_lora] */
} FstMlaCompressor;
int fst_cuda_mla_set_layer_compressor(FstMlaCtx* ctx, int lid, const FstMlaCompressor* w);
/* The compressed rows of a sequence in one layer [n, kv_lora] to host; rows == NULL: only the count. */
int fst_cuda_mla_cmp_read(FstMlaCtx* ctx, int lid, int32_t seq, uint16_t* rows, int32_t cap, int32_t* n_out);
/* Saves the compressor window state of a sequence (all layers) at its present length: a later
 * fst_cuda_mla_seq_truncate to exactly that length restores it, as the reference restores its
 * snapshot when it rejects speculative rows (src/fst_engine.cpp:6149-6152). */
int fst_cuda_mla_seq_snapshot(FstMlaCtx* ctx, int32_t seq);

/* ---- paged latent cache --------------------------------------------------------------- */
/* The reference cache is one flat [max_seq, 512] bf16 buffer per layer indexed by seq_pos_
 * (include/fst_engine.h:108-113; alloc src/fst_engine.cpp:1469-1474).  Here token t of a
 * sequence lives in page table[t / page_tokens], slot t % page_tokens, of every layer's
 * pool; pages come from a LIFO free list that initially hands out 0, 1, 2, ... */
int fst_cuda_mla_seq_alloc(FstMlaCtx* ctx, int32_t* seq_out);
int fst_cuda_mla_seq_free(FstMlaCtx* ctx, int32_t seq);
/* Grow the table to hold n_tokens (no-op if it already does). */
int fst_cuda_mla_seq_reserve(FstMlaCtx* ctx, int32_t seq, int32_t n_tokens);
/* Speculative-decoding rollback (src/fst_engine.cpp:6132-6147): drop rows >= n_tokens,
 * zero them in every layer as the reference does, return whole pages to the pool. */
int fst_cuda_mla_seq_truncate(FstMlaCtx* ctx, int32_t seq, int32_t n_tokens);
int fst_cuda_mla_seq_len(FstMlaCtx* ctx, int32_t seq, int32_t* len_out);
/* reset_session (src/fst_engine.cpp:2992-3012): free every sequence, zero the pools. */
int fst_cuda_mla_reset(FstMlaCtx* ctx);
int fst_cuda_mla_block_table(FstMlaCtx* ctx, int32_t seq, int32_t* out, int32_t cap, int32_t* n_out);
int fst_cuda_mla_free_pages(FstMlaCtx* ctx, int32_t* n_out);
/* Element offset of row `pos` of `seq` inside a layer's pool (page * page_tokens + slot) * row. */
int fst_cuda_mla_row_offset(FstMlaCtx* ctx, int32_t seq, int32_t pos, int64_t* off_out);
/* Copy n rows [n, row] starting at row pos0 from / to host memory (reserves pages on write). */
int fst_cuda_mla_cache_write(FstMlaCtx* ctx, int lid, int32_t seq, int32_t pos0, int32_t n,
                             const uint16_t* rows);
int fst_cuda_mla_cache_read(FstMlaCtx* ctx, int lid, int32_t seq, int32_t pos0, int32_t n,
                            uint16_t* rows);
/* Raw pool of a layer [n_pages * page_tokens, row] to host. */
int fst_cuda_mla_pool_read(FstMlaCtx* ctx, int lid, uint16_t* out, size_t bytes);

/* ---- the layer ------------------------------------------------------------------------ */
/* Host-side preparation of one call shape: reserves pages, builds block tables, RoPE tables
 * and the split-KV schedule, and uploads them.  A plan stays valid for every layer of the
 * same step (process_layer calls process_mla once per layer with the same seq_pos_). */
int fst_cuda_mla_plan(FstMlaCtx* ctx, const FstMlaSeqStep* steps, int32_t n_seqs, int32_t causal);
/* A plan request equal to the valid plan (same steps, same causal flag, no sequence touched in
 * between) returns at once and keeps the tables that are on the device: that is what layers
 * 2 .. L of a step see, also through fst_cuda_mla_forward.  on = 0 rebuilds every time. */
int fst_cuda_mla_set_plan_reuse(FstMlaCtx* ctx, int32_t on);
/* A query token whose whole context the split-KV schedule gives to ONE thread block needs no
 * merge: the attention kernel normalises, rounds and writes its output rows itself, no partial
 * goes to memory, and the merge kernel skips the token (and is not launched when every token is
 * such a token: verify blocks and prefill chunks mostly are).  on = 0: every token goes through
 * its partial and the merge kernel.  Both give the same bits.  Default: on. */
int fst_cuda_mla_set_fused_merge(FstMlaCtx* ctx, int32_t on);
/* Calls in which every sequence brings the same number G >= 4 of new tokens (speculative-verify
 * blocks, prefill chunks over a long context; the engine's M_PAD = 16 rows per call,
 * src/fst_engine.cpp:2959, 3573-3589) are scheduled by BLOCKS: the thread blocks form n_sm / G
 * groups of G lanes, the page columns of the sequences are cut into one run per group, and lane i
 * walks its group's run for token i -- so the G tokens of a sequence read each cache page at the
 * same time and it comes from HBM once, not G times.  on = 0: the token-by-token schedule of
 * decode for every call.  Results do not depend on it beyond the order of a token's parts.
 * Default: on. */
int fst_cuda_mla_set_block_schedule(FstMlaCtx* ctx, int32_t on);
/* Sliding window that fst_cuda_mla_forward applies to every sequence of its calls (0: none). */
int fst_cuda_mla_set_window(FstMlaCtx* ctx, int32_t window);
/* Plans built and plan requests answered by the valid plan, since the context was created. */
int fst_cuda_mla_plan_counts(FstMlaCtx* ctx, int64_t* built, int64_t* reused);
/* Enqueue the layer for the current plan; h_in / h_out are device bf16 [T, hidden]
 * (may alias).  No host synchronisation. */
int fst_cuda_mla_run_device(FstMlaCtx* ctx, int lid, const void* d_h_in, void* d_h_out);
/* process_mla with host buffers, as the engine calls it: plan + H2D + run + D2H + sync.
 * h_in / h_out are host bf16 [sum q_lens, hidden] (may alias: the reference works in place,
 * src/fst_engine.cpp:3889).  Rows are written at pos0[b] .. pos0[b]+q_lens[b]-1.
 * Page-locked buffers (cudaHostAlloc / cudaHostRegister) are copied directly; pageable ones
 * go through a page-locked staging buffer of the context, which costs two extra memcpy.  A
 * page-locked h_out that the device can address (cudaHostAlloc memory is) receives its rows
 * from the last GEMM itself, with no copy behind the layer. */
int fst_cuda_mla_forward(FstMlaCtx* ctx, int lid, const uint16_t* h_in, uint16_t* h_out,
                         const int32_t* seq_ids, const int32_t* pos0, const int32_t* q_lens,
                         int32_t n_seqs, int32_t causal);
/* QK / softmax / SV alone on caller-supplied queries (the qksv dispatches,
 * src/fst_engine.cpp:3588, 3682): host q_eff [T*H, d_qk] -> host o_lat [T*H, d_v], over the
 * cache as it stands, for the current plan (nothing is appended). */
int fst_cuda_mla_attention_only(FstMlaCtx* ctx, int lid, const uint16_t* q_eff, uint16_t* o_lat);
/* Split-KV across GPUs: run the layer up to the merged per-GPU partial.  d_partial is device
 * fp32 [T*H, 2 + d_v] holding (max, sum, un-normalised O) per query row. */
int fst_cuda_mla_run_partial_device(FstMlaCtx* ctx, int lid, const void* d_h_in, void* d_partial);
/* Merge n_parts gathered partials [n_parts][T*H, 2 + d_v] by log-sum-exp, then run the
 * output projections into d_h_out. */
int fst_cuda_mla_run_merge_device(FstMlaCtx* ctx, int lid, const void* d_partials, int32_t n_parts,
                                  void* d_h_out);
/* ---- split-KV across GPUs, exchange included -------------------------------------------------
 * One long sequence, its cache cut along the KV axis into one slice per GPU (one context per GPU,
 * one process per GPU or one process for all).  A layer call is: every GPU runs the front of the
 * layer and attends to its slice (as fst_cuda_mla_run_partial_device), ONE all-gather exchanges the
 * per-GPU (max, sum, un-normalised O) partials -- T*H rows of 2 + d_v floats per GPU, 131.6 KB for
 * one query token -- and every GPU merges them by log-sum-exp and runs the output projections.  The
 * reference has no counterpart (one NPU, 128 rows); the engine-side call is FSTEngine::process_mla_split.
 *
 * The transport is NCCL (ncclAllGather on the context's stream; no kernel reads another GPU's
 * memory), or a function the host supplies.  NCCL is not linked: the library already loaded in the
 * process is used, else libnccl.so.2 is opened when the first of these calls needs it. */
/* The 128 bytes every rank needs to join (ncclGetUniqueId); rank 0 creates them, the host hands
 * them to the other ranks by whatever means it has. */
int fst_cuda_mla_comm_unique_id(uint8_t id_out[128]);
/* Joins the context to a communicator of `world` ranks as rank `rank` (ncclCommInitRank on the
 * context's device; collective: every rank calls it) and allocates the exchange buffers. */
int fst_cuda_mla_comm_init(FstMlaCtx* ctx, const uint8_t id[128], int32_t rank, int32_t world);
/* A host-supplied transport instead: gather(user, d_send, d_recv, bytes_per_rank, cuda_stream) must
 * leave rank r's bytes at d_recv + r * bytes_per_rank on every rank, ordered on cuda_stream, and
 * return 0.  For hosts with their own collective layer, and for tests on one GPU. */
typedef int (*FstMlaGatherFn)(void* user, const void* d_send, void* d_recv, size_t bytes_per_rank, void* cuda_stream);
int fst_cuda_mla_comm_set_gather(FstMlaCtx* ctx, FstMlaGatherFn fn, void* user, int32_t rank, int32_t world);
int fst_cuda_mla_comm_destroy(FstMlaCtx* ctx);
/* The layer call for the current plan (the plan of a KV slice: FstMlaSeqStep.append = 1 on the rank
 * that owns the new rows, 0 elsewhere; rope_pos0 = the global position).  Device buffers as for
 * fst_cuda_mla_run_device; enqueued on the context's stream, no host synchronisation. */
int fst_cuda_mla_run_split_device(FstMlaCtx* ctx, int lid, const void* d_h_in, void* d_h_out);
/* The same with host buffers, as the engine calls it: plan (the steps of this GPU's slice) + H2D +
 * the split layer call + D2H + sync.  h_in / h_out: host bf16 [sum q_len, hidden], may alias. */
int fst_cuda_mla_forward_split(FstMlaCtx* ctx, int lid, const uint16_t* h_in, uint16_t* h_out,
                               const FstMlaSeqStep* steps, int32_t n_seqs, int32_t causal);

/* Number of new tokens T of the current plan. */
int fst_cuda_mla_plan_tokens(FstMlaCtx* ctx, int32_t* t_out);
int fst_cuda_mla_get_stage(FstMlaCtx* ctx, int stage, uint16_t* host_out, size_t bytes);

/* ---- GEMM tile engine alone ----------------------------------------------------------- */
/* npu_gemm_mla_vec (src/fst_engine.cpp:465-575): C[M,N] = A[M,K] * B[N,K]^T (b_kn = 0, the
 * b_col_maj kernels) or A[M,K] * B[K,N] (b_kn = 1, the b_row_maj qksv kernel); host bf16
 * buffers, fp32 accumulation.  The random-matrix probe of randmat_test (586-685) runs
 * through this. */
int fst_cuda_mla_gemm(FstMlaCtx* ctx, uint16_t* C, const uint16_t* A, const uint16_t* B, int M,
                      int N, int K, int b_kn);

/* ---- measurement ---------------------------------------------------------------------- */
/* Kernels launched by this context so far. */
int fst_cuda_mla_launch_count(FstMlaCtx* ctx, int64_t* n_out);
/* on != 0: bracket every kernel of a run with CUDA events on the context's stream. */
int fst_cuda_mla_set_profiling(FstMlaCtx* ctx, int on);
/* Synchronises, then returns the summed device time (ms) and launch count per
 * FST_MLA_K_* since the last call; ms_out / n_out have FST_MLA_K_COUNT entries. */
int fst_cuda_mla_kernel_times(FstMlaCtx* ctx, float* ms_out, int32_t* n_out);
/* Schedule of the current plan: partial count, CTAs of the attention kernel, cached rows read. */
int fst_cuda_mla_plan_info(FstMlaCtx* ctx, int32_t* n_partials, int32_t* n_ctas, int64_t* kv_rows);

/* GEMM and attention launches so far by kernel family: tcgen05 kernels, CUDA-core kernels.
 * FST_MLA_IMPL_AUTO takes the CUDA-core kernels for shapes the tcgen05 kernels do not cover
 * (head count other than 64, pages other than 64 tokens, unaligned rows); a benchmark prints
 * these so that the slow family can never be measured unnoticed. */
int fst_cuda_mla_family_counts(FstMlaCtx* ctx, int64_t* tensor_out, int64_t* simt_out);

/* ---- robustness checks ------------------------------------------------------------------ */
/* Every wait inside the kernels is bounded: a kernel that gives one up records a status word,
 * lets its copies land, frees its tensor memory and returns; the next fst_cuda_mla_sync then
 * returns FST_MLA_ERR_DEVICE_CHECK and clears the word, and the context stays usable.  This call
 * exercises that path without touching the product kernels: one tiny kernel (no TMA, no MMA, no
 * tensor memory) waits on a barrier that nothing arrives at, with a limit of `polls` polls
 * (1 .. 65536), gives up and records its status.  Enqueued on the context's stream. */
int fst_cuda_mla_selftest_wait_expiry(FstMlaCtx* ctx, int32_t polls);
/* The split-KV schedule of a call, cut on the host without any device (for tests of the cutting
 * rules): sequences b = 0 .. n_seqs-1 bring q_lens[b] new rows at pos0[b]; a row sees [0, pos0 + i + 1)
 * when causal, [0, pos0 + q_len) otherwise; n_sm thread blocks; by_blocks allows the block schedule
 * (fst_cuda_mla_set_block_schedule).  segs_out receives five values per segment, in the order the
 * thread blocks walk them: token, first row, end row, partial slot, thread block.
 * *cut_by_blocks_out tells which rule cut it. */
int fst_cuda_mla_debug_schedule(int32_t n_sm, const int32_t* pos0, const int32_t* q_lens, int32_t n_seqs, int32_t causal,
                                int32_t by_blocks, int32_t* segs_out, int32_t cap, int32_t* n_segs_out,
                                int32_t* n_ctas_out, int32_t* cut_by_blocks_out);
/* Test hook: writes `code` into the device status word, as a kernel that failed a check would. */
int fst_cuda_mla_debug_set_status(FstMlaCtx* ctx, int32_t code);
/* Test hook, host only (no CUDA call): the library sets function attributes (the dynamic
 * shared-memory limit, the carve-out preference) once per (kernel, device), because they belong
 * to the device that is current when they are set.  Returns 1 the first time the triple
 * (kernel_key, device, value) is seen -- and again when a later value is larger -- else 0. */
int fst_cuda_mla_debug_attr_first_use(uint64_t kernel_key, int32_t device, int64_t value);

/* ---- decode attention without any allocation -------------------------------------------- */
/* No counterpart in the reference.  For callers that cannot allocate device memory at the
 * moment they need attention: a serving process whose device memory was handed out in full at
 * start-up, a latency-critical callback where cudaMalloc (which synchronises the device) is not
 * allowed, a plugin that only receives device pointers.  It needs no FstMlaCtx and calls no
 * cudaMalloc / cudaFree nor any allocating library routine.
 *
 * One query token: d_q_eff device bf16 [n_heads, d_qk]; d_cache device bf16 [n_rows, d_qk],
 * contiguous rows whose stride is exactly d_qk elements (no padding between rows),
 * keys = row[:d_qk], values = row[:d_v]; d_o_lat device bf16 [n_heads, d_v]
 * = softmax(scale * q K^T) V, no sink.  Both inputs 16-byte aligned.  Work is enqueued on
 * cuda_stream (NULL: default stream) of the current device; the call does not synchronise.
 *
 * The split-KV partials live in a fixed array inside the library image (about 4 MiB, held by
 * every GPU that loads the library until the process exits), hence the limits: n_rows <= 65536,
 * n_heads <= 64, d_qk <= 576 (multiple of 8), d_v <= 512 (multiple of 64, <= d_qk).  Anything
 * larger returns FST_MLA_ERR_CAPACITY (fst_cuda_mla_last_error says why); use the context API
 * then.  A CUDA error that an earlier call left pending on the calling thread is reported as
 * FST_MLA_ERR_CUDA without being cleared, and nothing is launched.
 * All calls share that one array: it keeps the previous call's contents, every call rewrites
 * whatever it later reads (nothing has to start at zero), and two calls that overlap on the
 * GPU -- different streams, or different host threads -- race on it.  Serialise them.
 * The full MLA shape (64 heads, d_qk 576 or 512, d_v 512, at least one 64-row page) runs the
 * tcgen05 streaming kernel on up to 32 thread blocks -- 75 us for 65536 rows; every other shape
 * the CUDA-core kernel.
 * The first call on a device looks up the array's device address, and the first call of a shape
 * class sets that kernel's attributes; make those first calls before any stream capture begins. */
int fst_cuda_mla_attention_noalloc(const void* d_q_eff, const void* d_cache, int32_t n_rows, int32_t n_heads,
                                   int32_t d_qk, int32_t d_v, float softmax_scale, void* d_o_lat,
                                   void* cuda_stream);

#ifdef __cplusplus
}
#endif
#endif
