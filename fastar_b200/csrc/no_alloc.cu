// Decode attention for callers that must not allocate device memory.
//
// Some hosts of this library cannot call cudaMalloc when they need an attention result: code
// that runs inside a memory-budgeted serving process whose device memory is fully handed out at
// start-up, a callback on a latency-critical thread where an allocation (a device-wide
// synchronisation point) is forbidden, or a plugin that only ever receives device pointers
// from its host.  The regular path keeps its split-KV partials in workspaces that
// fst_cuda_mla_create allocates; this entry point keeps them in a fixed array that is part of
// the library image instead, so it needs no context and allocates nothing, at the price of a
// stated maximum problem size.
#include <algorithm>
#include <cmath>
#include <cstdio>

#include "../../include/fst_cuda_mla.h"
#include "kernels.cuh"

using namespace fst;

namespace {

constexpr int NA_MAX_ROWS = 65536;   // cached rows
constexpr int NA_MAX_HEADS = 64;
constexpr int NA_MAX_DV = 512;
constexpr int NA_MAX_DQK = 576;
constexpr int NA_MAX_SPLITS = 32;    // KV splits = thread blocks of the attention kernel
constexpr int NA_PAGE = 64;

// Layout of the scratch array (byte offsets, all multiples of 256).
constexpr size_t OFF_PART_O = 0;
constexpr size_t SZ_PART_O = (size_t)NA_MAX_SPLITS * NA_MAX_HEADS * NA_MAX_DV * sizeof(float);  // 4 MiB
constexpr size_t OFF_PART_M = OFF_PART_O + SZ_PART_O;
constexpr size_t SZ_PART_ML = (size_t)NA_MAX_SPLITS * NA_MAX_HEADS * sizeof(float);
constexpr size_t OFF_PART_L = OFF_PART_M + SZ_PART_ML;
constexpr size_t OFF_SEGS = OFF_PART_L + SZ_PART_ML;
constexpr size_t OFF_TABLE = OFF_SEGS + 1024;                                   // 32 segments x 20 bytes, padded
constexpr size_t OFF_TOK = OFF_TABLE + (NA_MAX_ROWS / NA_PAGE) * sizeof(int32_t);  // tok_table[1], tok_part[2]; from
                                                                                // int 16: cta_seg[33]; int 60: status
constexpr size_t OFF_LUT = OFF_TOK + 256;                                       // unused RoPE table slot
constexpr size_t SCRATCH_BYTES = OFF_LUT + 256;

// Every GPU that loads the library holds this array (about 4.02 MiB) until the process exits.
static __device__ __align__(256) unsigned char g_na_scratch[SCRATCH_BYTES];

// Device address of g_na_scratch per device.  In host code the array's name is only a
// stand-in for the symbol, not an address a kernel could use: the address comes from
// cudaGetSymbolAddress, asked once per device with that device current.
unsigned char* g_na_ptr[64] = {nullptr};

// Rewrites every piece of bookkeeping the attention and merge kernels read from the scratch:
// an identity block table (the cache is contiguous), the split schedule, the one-token maps.
// unit: rows per schedule tile -- 32 for the CUDA-core kernel, 64 (a page) for the tcgen05 one,
// whose thread block k walks segment k (cta_seg) and reports a wait that ran out in the status word.
__global__ void k_na_setup(unsigned char* scratch, int n_rows, int n_splits, int unit) {
  AttnSeg* segs = reinterpret_cast<AttnSeg*>(scratch + OFF_SEGS);
  int32_t* table = reinterpret_cast<int32_t*>(scratch + OFF_TABLE);
  int32_t* tok = reinterpret_cast<int32_t*>(scratch + OFF_TOK);
  const int n_pages = (n_rows + NA_PAGE - 1) / NA_PAGE;
  for (int i = threadIdx.x; i < n_pages; i += blockDim.x) table[i] = i;
  if (threadIdx.x < n_splits) {
    // equal runs of tiles; the last split takes the ragged end
    const int tiles = (n_rows + unit - 1) / unit;
    const int s = threadIdx.x;
    AttnSeg sg;
    sg.tok = 0;
    sg.kv_begin = (int)((long long)tiles * s / n_splits) * unit;
    sg.kv_end = min(n_rows, (int)((long long)tiles * (s + 1) / n_splits) * unit);
    sg.part = s;
    sg.table = 0;  // the identity block table starts at entry 0
    segs[s] = sg;
  }
  if (threadIdx.x <= n_splits) tok[16 + threadIdx.x] = threadIdx.x;  // cta_seg: block k takes segment k
  if (threadIdx.x == 0) {
    tok[0] = 0;         // tok_table[0]: the token's block table starts at entry 0
    tok[1] = 0;         // tok_part[0]
    tok[2] = n_splits;  // tok_part[1]
    tok[60] = 0;        // status word of the bounded waits
  }
}

// Failures are reported like those of every other entry point: the message goes to the calling
// thread's last-error string (fst_cuda_mla_last_error).
int na_fail(int code, const char* msg) {
  char buf[256];
  snprintf(buf, sizeof(buf), "fst_cuda_mla_attention_noalloc: %s", msg);
  set_last_error(buf);
  return code;
}

}  // namespace

extern "C" int fst_cuda_mla_attention_noalloc(const void* d_q_eff, const void* d_cache, int32_t n_rows,
                                              int32_t n_heads, int32_t d_qk, int32_t d_v, float softmax_scale,
                                              void* d_o_lat, void* cuda_stream) {
  if (!d_q_eff || !d_cache || !d_o_lat) return na_fail(FST_MLA_ERR_ARG, "null device pointer");
  if (n_rows <= 0 || n_heads <= 0 || d_qk <= 0 || d_v <= 0)
    return na_fail(FST_MLA_ERR_ARG, "non-positive size");
  if (!(softmax_scale > 0.0f) || !std::isfinite(softmax_scale))  // also rejects NaN
    return na_fail(FST_MLA_ERR_ARG, "softmax_scale must be a positive finite number");
  if (n_rows > NA_MAX_ROWS || n_heads > NA_MAX_HEADS || d_v > NA_MAX_DV || d_qk > NA_MAX_DQK)
    return na_fail(FST_MLA_ERR_CAPACITY,
                   "beyond the fixed scratch: at most 65536 cached rows, 64 heads, d_qk 576, d_v 512");
  if (d_qk % 8 || d_v % 64 || d_v > d_qk)
    return na_fail(FST_MLA_ERR_ARG, "d_qk must be a multiple of 8, d_v a multiple of 64 and <= d_qk");
  if ((reinterpret_cast<uintptr_t>(d_q_eff) & 15) || (reinterpret_cast<uintptr_t>(d_cache) & 15))
    return na_fail(FST_MLA_ERR_ARG, "q_eff and cache must be 16-byte aligned");
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess) return na_fail(FST_MLA_ERR_NO_DEVICE, "no current CUDA device");
  // An error left pending by an earlier call of the caller's is the caller's to read: it is
  // reported here but not cleared, and nothing is launched on top of it.
  if (cudaPeekAtLastError() != cudaSuccess)
    return na_fail(FST_MLA_ERR_CUDA, "a CUDA error from an earlier call is pending on this thread; nothing was launched");
  if (dev < 0 || dev >= 64) return na_fail(FST_MLA_ERR_ARG, "device ordinal out of range");
  if (!g_na_ptr[dev]) {
    // first call on this device: resolve the device address of the scratch array
    void* p = nullptr;
    cudaError_t e = cudaGetSymbolAddress(&p, g_na_scratch);
    if (e != cudaSuccess || !p) {
      cudaGetLastError();
      return na_fail(FST_MLA_ERR_CUDA, cudaGetErrorString(e));
    }
    g_na_ptr[dev] = static_cast<unsigned char*>(p);
  }
  unsigned char* sc = g_na_ptr[dev];
  cudaStream_t st = static_cast<cudaStream_t>(cuda_stream);
  AttnArgs a;
  a.q_eff = static_cast<const bf16*>(d_q_eff);
  a.pool = static_cast<const bf16*>(d_cache);
  a.tables = reinterpret_cast<const int32_t*>(sc + OFF_TABLE);
  a.segs = reinterpret_cast<const AttnSeg*>(sc + OFF_SEGS);
  a.cta_seg = reinterpret_cast<const int32_t*>(sc + OFF_TOK) + 16;
  a.part_m = reinterpret_cast<float*>(sc + OFF_PART_M);
  a.part_l = reinterpret_cast<float*>(sc + OFF_PART_L);
  a.part_o = reinterpret_cast<float*>(sc + OFF_PART_O);
  a.d_status = reinterpret_cast<int*>(sc + OFF_TOK) + 60;
  a.H = n_heads;
  a.d_qk = d_qk;
  a.d_v = d_v;
  a.row = d_qk;
  a.page_tokens = NA_PAGE;
  a.q_rows = n_heads;
  a.pool_rows = n_rows;
  a.scale = softmax_scale;
  // The full MLA shape (64 heads, 576- or 512-wide rows, 512 value columns) goes to the tcgen05
  // streaming kernel, one thread block per split over whole 64-row pages; every other shape to the
  // CUDA-core kernel (so do caches of less than one page).  Either way at most 32 splits: that is
  // what the scratch holds.
  const bool stream = n_rows >= NA_PAGE && attn_stream_supported(a);
  const int unit = stream ? NA_PAGE : 32;
  const int n_splits = std::max(1, std::min(NA_MAX_SPLITS, stream ? (n_rows + NA_PAGE - 1) / NA_PAGE : (n_rows + 127) / 128));
  a.n_segs = n_splits;
  a.n_ctas = n_splits;
  k_na_setup<<<1, 256, 0, st>>>(sc, n_rows, n_splits, unit);
  if (stream) {
    // (not as a programmatic dependent: the schedule it reads on entry was written by k_na_setup)
    a.dependent_launch = false;
    cudaError_t es = launch_attn_stream(a, st);
    if (es != cudaSuccess) return na_fail(FST_MLA_ERR_CUDA, cudaGetErrorString(es));
  } else {
    launch_attn_simt(a, st);
  }

  MergeArgs m;
  m.part_m = a.part_m;
  m.part_l = a.part_l;
  m.part_o = a.part_o;
  m.tok_part = reinterpret_cast<const int32_t*>(sc + OFF_TOK) + 1;
  m.sinks = nullptr;
  m.lut = reinterpret_cast<const float*>(sc + OFF_LUT);
  m.o_lat = static_cast<bf16*>(d_o_lat);
  m.rank_partial = nullptr;
  m.T = 1;
  m.H = n_heads;
  m.d_v = d_v;
  m.rope = 0;
  m.inv_rope = 0;
  m.mode = 0;
  m.threads = 256;
  m.wide = 1;  // one query token: a block per (head row, 128 columns) where the shape allows
  launch_merge(m, st);
  cudaError_t e = cudaGetLastError();
  if (e != cudaSuccess) return na_fail(FST_MLA_ERR_CUDA, cudaGetErrorString(e));
  return FST_MLA_OK;
}
