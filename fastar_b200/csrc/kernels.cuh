// Launchers of the MLA kernels.  All pointers are device pointers; bf16 unless noted.
#pragma once
#include <map>
#include <mutex>
#include <utility>
#include "common.cuh"

namespace fst {

// Function attributes (the dynamic shared-memory limit, the carve-out preference) belong to the
// DEVICE that is current when they are set, so a process that drives several GPUs has to set
// them once per (kernel, device).  This is the bookkeeping: first_use() answers true exactly once
// for every (kernel, device ordinal, value) triple -- a larger value asked for later answers true
// again.  Pure host logic (no CUDA call), so it can be checked without a GPU.
class PerDeviceOnce {
 public:
  bool first_use(const void* kernel, int device, long long value = 0) {
    std::lock_guard<std::mutex> lk(mu_);
    auto key = std::make_pair(kernel, device);
    auto it = seen_.find(key);
    if (it != seen_.end() && it->second >= value) return false;
    seen_[key] = value;
    return true;
  }

 private:
  std::mutex mu_;
  std::map<std::pair<const void*, int>, long long> seen_;
};
PerDeviceOnce& kernel_attr_registry();

inline int current_device() {
  int dev = 0;
  cudaGetDevice(&dev);
  return dev;
}

// Raises the dynamic shared-memory limit of `kernel` to `bytes` on the current device (once per
// device; again when a later launch needs more).
inline cudaError_t ensure_dynamic_smem(const void* kernel, size_t bytes) {
  if (bytes <= 48 * 1024) return cudaSuccess;
  if (!kernel_attr_registry().first_use(kernel, current_device(), (long long)bytes)) return cudaSuccess;
  return cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)bytes);
}

// Every kernel of the library asks for the largest shared-memory carve-out, whatever it uses:
// an SM that has to change its L1 / shared split between two kernels drains first, and the
// attention kernel (227 KB) would pay that after every GEMM.  Once per kernel and device.
inline void prefer_max_shared(const void* kernel) {
  // (the tag keeps this entry apart from the kernel's dynamic shared-memory entry)
  if (kernel_attr_registry().first_use(static_cast<const char*>(kernel) + 1, current_device()))
    cudaFuncSetAttribute(kernel, cudaFuncAttributePreferredSharedMemoryCarveout, cudaSharedmemCarveoutMaxShared);
}

// Launch with programmatic stream serialisation (and an optional cluster along y).
template <class... KArgs, class... Args>
inline cudaError_t launch_k(bool dependent, void (*kernel)(KArgs...), dim3 grid, dim3 block, size_t smem, cudaStream_t st,
                            int cluster_y, Args&&... args) {
  prefer_max_shared(reinterpret_cast<const void*>(kernel));
  cudaError_t e_attr = ensure_dynamic_smem(reinterpret_cast<const void*>(kernel), smem);
  if (e_attr != cudaSuccess) return e_attr;
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = grid;
  cfg.blockDim = block;
  cfg.dynamicSmemBytes = smem;
  cfg.stream = st;
  cudaLaunchAttribute attr[2];
  int n = 0;
  if (dependent) {
    attr[n].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[n].val.programmaticStreamSerializationAllowed = 1;
    ++n;
  }
  if (cluster_y > 1) {
    attr[n].id = cudaLaunchAttributeClusterDimension;
    attr[n].val.clusterDim.x = 1;
    attr[n].val.clusterDim.y = cluster_y;
    attr[n].val.clusterDim.z = 1;
    ++n;
  }
  cfg.attrs = attr;
  cfg.numAttrs = n;
  return cudaLaunchKernelEx(&cfg, kernel, static_cast<KArgs>(args)...);
}
// Programmatic dependent launch: the kernel may start while its predecessor in the stream drains
// and orders itself behind it with griddepcontrol.wait.
template <typename... KArgs, typename... Args>
inline cudaError_t launch_pdl(void (*kernel)(KArgs...), dim3 grid, dim3 block, size_t smem, cudaStream_t st,
                              int cluster_y, Args&&... args) {
  return launch_k(true, kernel, grid, block, smem, st, cluster_y, static_cast<Args&&>(args)...);
}

// Strided-batched C[z][m, n] = sum_k A[z][m, k] * B[z][n, k]  (b_kn: B[z][k, n]).
struct GemmArgs {
  const bf16* A;
  const bf16* B;
  bf16* C;
  int M, N, K;
  int lda, ldb, ldc;
  int batch;
  long long a_bs, b_bs, c_bs;  // element strides between batch members
  int b_kn;
  // Optional side job of the tcgen05 kernel (null: none): while the tensor pipe works, the idle
  // epilogue warps of batch member z's first CTA rotate the rope pairs of head z for every
  // token: src[(t*H + z)*q_head + nope + 2p ..] -> dst[(t*H + z)*d_qk + d_qk - rope + 2p ..].
  // This is the BASELINE q_pe RoPE (reference src/fst_engine.cpp:2025-2058), which depends on
  // the same input as the absorb GEMM and writes other columns of the same output.
  const bf16* rope_src = nullptr;
  const float* rope_lut = nullptr;  // [T, rope] (cos, sin) pairs
  bf16* rope_dst = nullptr;
  int rope_T = 0, rope_H = 0, rope_q_head = 0, rope_nope = 0, rope_dims = 0, rope_d_qk = 0;
  // Optional, tcgen05 kernel only (null: off): every block, as its last act, reads the device status
  // word of the bounded waits and, if it is not zero, stores it to *status_host -- a word in
  // page-locked host memory that the device can address.  Given to the LAST kernel of a layer call:
  // the host then has the status when the stream is synchronised, without a copy behind the call.
  const int* status_dev = nullptr;
  int* status_host = nullptr;
};
void launch_gemm_simt(const GemmArgs& g, cudaStream_t st);
// tcgen05 path: B in [N, K] layout only, K % 64 == 0, N % 128 == 0, 16-byte aligned rows.
bool gemm_tc_supported(const GemmArgs& g);
// Returns cudaSuccess or the error of building the tensor maps / launching.
cudaError_t launch_gemm_tc(const GemmArgs& g, int* d_status, cudaStream_t st);

// y[t] = x[t] * w / sqrt(mean(x[t]^2) + eps) over `dim` (<= 8192) elements, rounded to bf16: the
// attn_norm of process_layer (reference src/fst_engine.cpp:2687-2688).
void launch_rmsnorm_rows(const bf16* x, const bf16* w, bf16* y, int T, int dim, float eps, cudaStream_t st);

// RMSNorm(q) -> qc; RMSNorm(latent) (+ RoPE on the key's rope dims) -> kv_new and the cache row.
struct NormAppendArgs {
  const bf16* cmp;      // [T, q_lora + row]
  const bf16* q_norm;   // [q_lora] or null
  const bf16* kv_norm;  // [kv_lora] or null
  const float* lut;     // [T, rope] (cos, sin) pairs
  const long long* dst_row;  // [T] element offset of the cache row in the pool, or -1
  bf16* qc;             // [T, q_lora]
  bf16* kv_new;         // [T, row]
  bf16* pool;
  int T, q_lora, kv_lora, row, rope;
  float eps;
};
void launch_norm_append(const NormAppendArgs& a, cudaStream_t st);

// BASELINE: rotate q_pe into q_eff[:, kv_lora:].  V4: per-head RMSNorm + tail RoPE -> q_eff.
struct QPrepArgs {
  const bf16* q_full;  // [T, H * q_head]
  const float* lut;    // [T, rope]
  bf16* q_eff;         // [T * H, d_qk]
  int T, H, q_head, nope, rope, d_qk, v4;
  float eps;
  // V4 only.  head_norm: the per-head weightless RMSNorm (reference 3487-3495); rope_heads: heads
  // 0 .. rope_heads-1 get their tail rotated.  The main model: 1 and all heads; the draft model's
  // layer has no head norm and rotates head 0 only (process_draft_mla, 4967-4983).
  int head_norm = 1, rope_heads = 1 << 30;
};
void launch_q_prep(const QPrepArgs& a, cudaStream_t st);

struct AttnArgs {
  const bf16* q_eff;        // [T * H, d_qk]
  const bf16* pool;         // [n_pages * page_tokens, row]
  const int32_t* tables;    // flat block tables (a segment names where its table starts)
  const AttnSeg* segs;
  const int32_t* cta_seg;   // [n_ctas + 1] segment ranges of the persistent CTAs
  float* part_m;            // [P, H]
  float* part_l;            // [P, H]
  float* part_o;            // [P, H, d_v]
  int* d_status;
  int n_segs, n_ctas, H, d_qk, d_v, row, page_tokens;
  long long q_rows;         // rows of q_eff (new tokens * H)
  long long pool_rows;      // n_pages * page_tokens
  float scale;
  // tcgen05 kernel: launch as a programmatic dependent of the kernel before it in the stream.  Off
  // for callers whose schedule arrays (segs, cta_seg, tables) are WRITTEN by that kernel: the
  // attention kernel reads its block's segment range before it waits for its predecessor.
  bool dependent_launch = true;
  // the schedule makes several thread blocks read the same cache tiles at about the same time
  // (blocks of query tokens): tiles then keep the normal L2 priority instead of leaving first, and
  // the tcgen05 kernel lets each QK issuer take whole tiles (k_attn_stream, WHOLE)
  bool tiles_shared = false;
  // tcgen05 kernel only: a token whose whole context is ONE segment of the schedule (one partial)
  // is normalised and written to o_lat by the attention kernel itself and leaves no partial; the
  // merge kernel that follows is told to skip such tokens (MergeArgs::skip_single).
  bool direct_single = false;
  const int32_t* tok_part = nullptr;  // [T + 1]
  bf16* o_lat = nullptr;              // [T * H, d_v]
  const float* sinks = nullptr;       // [H] or null
  const float* lut = nullptr;         // [T, rope]
  int rope = 0, inv_rope = 0;           // inv_rope: heads 0 .. inv_rope-1 get the inverse rotation of their output tail
};
void launch_attn_simt(const AttnArgs& a, cudaStream_t st);
// tcgen05 kernel: a stream of 64-token tiles, Q_eff in tensor memory, ring of three tile frames.
bool attn_stream_supported(const AttnArgs& a);
cudaError_t launch_attn_stream(const AttnArgs& a, cudaStream_t st);

// Log-sum-exp merge of each token's partial slots [tok_part[t], tok_part[t+1]).
struct MergeArgs {
  const float* part_m;
  const float* part_l;
  const float* part_o;
  const int32_t* tok_part;  // [T + 1]
  const float* sinks;       // [H] or null
  const float* lut;         // [T, rope]: inverse RoPE of the output tail of heads 0 .. inv_rope-1
  bf16* o_lat;              // [T * H, d_v]                 (mode 0)
  float* rank_partial;      // [T * H, 2 + d_v] fp32        (mode 1, no sink)
  int T, H, d_v, rope, inv_rope, mode;
  int threads;              // 128: rows have few parts (a thread per 4 columns); otherwise 256 (8 warps share the parts)
  int skip_single = 0;      // rows of tokens with exactly one partial are already in o_lat (AttnArgs::direct_single)
  int wide = 0;             // few rows with many parts each: a block per (row, 128 columns) instead of per row
};
void launch_merge(const MergeArgs& a, cudaStream_t st);

// Merge of gathered per-GPU partials [n_parts][T * H, 2 + d_v] -> o_lat.
struct MergeGatheredArgs {
  const float* parts;
  const float* sinks;
  const float* lut;
  bf16* o_lat;
  int n_parts, T, H, d_v, rope, inv_rope;
};
void launch_merge_gathered(const MergeGatheredArgs& a, cudaStream_t st);

// Robustness self-test: one block waits on an mbarrier nothing ever arrives at, with a limit of
// `polls` polls, gives up and records ST_SELFTEST_TIMEOUT in *d_status the way the tcgen05 kernels
// record their own time-outs.  No TMA, no MMA, no tensor memory.
void launch_wait_selftest(int* d_status, uint32_t polls, cudaStream_t st);

// The calling thread's last-error string (what fst_cuda_mla_last_error returns).
void set_last_error(const char* msg);

// V4 KV compressor (reference compress_token, src/fst_engine.cpp:3171-3318) for the new rows of a
// layer call, one thread block per sequence, its rows in order: gate bias, window state, and on
// every ratio-th position the pooled / normed / tail-rotated / E4M3-round-tripped row, written to
// the compressed-row pages.
struct CompressTok {
  long long dst;   // element offset of the compressed row this token emits in the pool, or -1
  int32_t pos;     // position of the token in its sequence
  int32_t pad;
};
struct CompressStep {
  int32_t tok0, q_len, slot;  // first row of the sequence in this call, rows, state slot of the sequence
  int32_t pad;
};
struct CompressArgs {
  const bf16* proj;          // [T, 2 * width]: wkv product then wgate product of every row
  const float* ape;          // [ratio, width]
  const bf16* norm;          // [kv_lora]
  const float* lut;          // [T, rope] (cos, sin) of the compressed position of an emitting row
  const CompressTok* toks;   // [T]
  const CompressStep* steps; // [n_steps]
  float* state;              // [slots][2][rows, width] window state (values, then scores)
  bf16* pool;
  int n_steps, ratio, width, kv_lora, rope;
};
void launch_compress(const CompressArgs& a, cudaStream_t st);

void launch_zero_rows(bf16* pool, const long long* row_off, int n_rows, int row, cudaStream_t st);

}  // namespace fst
