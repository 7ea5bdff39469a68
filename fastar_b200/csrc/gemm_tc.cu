// Skinny bf16 GEMM on the 5th-generation tensor cores: C[M, N] = A[M, K] * W[N, K]^T with the
// weight rows as the MMA M dimension (128 per CTA) and the tokens as the MMA N dimension, so a
// handful of tokens still fills a full-rate 128-row tcgen05.mma.  This is the tile engine the
// reference calls npu_gemm_mla_vec (src/fst_engine.cpp:465-575): weights stay in their native
// [N, K] layout and are streamed from HBM exactly once.
//
// One CTA = one (128-row weight tile, token tile, K split).  Warp 0 streams both operands with
// TMA through a ring of 128-byte-swizzled stages; one lane of warp 1 issues tcgen05.mma into
// a TMEM accumulator; warps 2-5 drain TMEM.  When K is split the CTAs leave fp32 partials and
// the last one to finish a tile adds them in split order (deterministic) and writes bf16.
#include <mutex>
#include <unordered_map>

#include "kernels.cuh"
#include "tc_common.cuh"

namespace fst {

namespace {

constexpr int BK = 64;          // K elements per stage: one 128-byte swizzle span
constexpr int W_TILE = 128;     // weight rows per CTA
constexpr int W_BYTES = W_TILE * BK * 2;
constexpr int GEMM_THREADS = 192;

struct GemmTcParams {
  bf16* C;
  float* ws;           // [batch][splits][M][N] fp32 partials (splits > 1)
  unsigned* counters;  // one per output tile, all zero between launches
  int* d_status;
  int M, N, K, ldc;
  long long c_bs;
  int splits, kc_total, stages;
  int w_swap, a_swap;  // the batch index is the middle tensor-map coordinate (its stride is the smaller one)
};

template <int NT>
__global__ void __launch_bounds__(GEMM_THREADS, 1)
k_gemm_tc(const __grid_constant__ CUtensorMap tmW, const __grid_constant__ CUtensorMap tmA, GemmTcParams p) {
  extern __shared__ __align__(1024) unsigned char smem_raw[];
  constexpr int A_BYTES = NT * BK * 2;
  constexpr int STAGE_BYTES = W_BYTES + A_BYTES;
  constexpr uint32_t TMEM_COLS = NT < 32 ? 32 : NT;
  unsigned char* smem = reinterpret_cast<unsigned char*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint64_t* full = reinterpret_cast<uint64_t*>(smem + (size_t)p.stages * STAGE_BYTES);
  uint64_t* empty = full + p.stages;
  uint64_t* acc_bar = empty + p.stages;
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(acc_bar + 1);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);
  int* last_flag = const_cast<int*>(abort_flag) + 1;

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int n0 = blockIdx.x * W_TILE;
  const int m_tile = blockIdx.y / p.splits, split = blockIdx.y % p.splits;
  const int m0 = m_tile * NT;
  const int z = blockIdx.z;
  const int kc0 = (int)((long long)p.kc_total * split / p.splits);
  const int kc1 = (int)((long long)p.kc_total * (split + 1) / p.splits);
  const int n_kc = kc1 - kc0;

  if (threadIdx.x == 0) {
    for (int s = 0; s < p.stages; ++s) {
      tc::mbar_init(&full[s], 1);
      tc::mbar_init(&empty[s], 1);
    }
    tc::mbar_init(acc_bar, 1);
    *abort_flag = 0;
    *last_flag = 0;
    tc::fence_barrier_init();
  }
  if (warp == 1) tc::tmem_alloc(tmem_slot, TMEM_COLS);
  tc::tc_fence_before();
  __syncthreads();
  tc::tc_fence_after();
  const uint32_t tmem = *tmem_slot;

  if (warp == 0) {
    if (lane == 0) {
      tc::tma_prefetch_desc(&tmW);
      tc::tma_prefetch_desc(&tmA);
      for (int i = 0; i < n_kc; ++i) {
        const int s = i % p.stages;
        if (i >= p.stages && !tc::mbar_wait(&empty[s], ((i / p.stages) - 1) & 1, abort_flag, p.d_status, ST_TMA_TIMEOUT))
          break;
        unsigned char* st = smem + (size_t)s * STAGE_BYTES;
        tc::mbar_expect_tx(&full[s], STAGE_BYTES);
        tc::tma_load_3d(st, &tmW, &full[s], (kc0 + i) * BK, p.w_swap ? z : n0, p.w_swap ? n0 : z);
        tc::tma_load_3d(st + W_BYTES, &tmA, &full[s], (kc0 + i) * BK, p.a_swap ? z : m0, p.a_swap ? m0 : z);
      }
    }
  } else if (warp == 1) {
    if (lane == 0) {
      constexpr uint32_t idesc = tc::umma_idesc_bf16(W_TILE, NT, 0, 0);
      bool ok = true;
      for (int i = 0; i < n_kc && ok; ++i) {
        const int s = i % p.stages;
        ok = tc::mbar_wait(&full[s], (i / p.stages) & 1, abort_flag, p.d_status, ST_MMA_TIMEOUT);
        if (!ok) break;
        tc::tc_fence_after();
        const uint32_t w_addr = tc::smem_u32(smem + (size_t)s * STAGE_BYTES);
        const uint32_t a_addr = w_addr + W_BYTES;
#pragma unroll
        for (int k = 0; k < BK / 16; ++k) {
          const uint64_t da = tc::umma_desc_sw128(w_addr + k * 32, 16, 1024);
          const uint64_t db = tc::umma_desc_sw128(a_addr + k * 32, 16, 1024);
          tc::umma_bf16(tmem, da, db, idesc, (i > 0 || k > 0) ? 1u : 0u);
        }
        tc::umma_commit(&empty[s]);  // the stage is free once these MMAs have read it
      }
      if (ok) tc::umma_commit(acc_bar);
    }
  } else {
    // epilogue warps: TMEM lane quadrant = warp % 4
    const int quad = warp & 3;
    const bool ok = n_kc == 0 || tc::mbar_wait(acc_bar, 0, abort_flag, p.d_status, ST_EPI_TIMEOUT);
    tc::tc_fence_after();
    const int n = n0 + quad * 32 + lane;
    if (ok) {
      for (int c0 = 0; c0 < NT; c0 += 32) {
        if (m0 + c0 >= p.M) break;
        float v[32];
        if (n_kc > 0) {
          tc::tmem_ld32(tmem + ((uint32_t)(quad * 32) << 16) + c0, v);
        } else {
#pragma unroll
          for (int j = 0; j < 32; ++j) v[j] = 0.0f;
        }
        if (n < p.N) {
          if (p.splits == 1) {
            bf16* c = p.C + z * p.c_bs + n;
#pragma unroll
            for (int j = 0; j < 32; ++j)
              if (j < NT - c0 && m0 + c0 + j < p.M) c[(long long)(m0 + c0 + j) * p.ldc] = f2bf(v[j]);
          } else {
            float* w = p.ws + (((long long)z * p.splits + split) * p.M) * p.N + n;
#pragma unroll
            for (int j = 0; j < 32; ++j)
              if (j < NT - c0 && m0 + c0 + j < p.M) w[(long long)(m0 + c0 + j) * p.N] = v[j];
          }
        }
      }
    }
  }

  // split-K: the CTA that finishes a tile last adds the partials in split order
  if (p.splits > 1) {
    __threadfence();
    __syncthreads();
    if (threadIdx.x == 0) {
      unsigned* ctr = p.counters + ((size_t)z * (gridDim.y / p.splits) + m_tile) * gridDim.x + blockIdx.x;
      const unsigned old = atomicAdd(ctr, 1u);
      if (old == (unsigned)p.splits - 1) {
        *last_flag = 1;
        *ctr = 0;
      }
    }
    __syncthreads();
    if (*last_flag) {
      __threadfence();
      const int mt = min(NT, p.M - m0), nt = min(W_TILE, p.N - n0);
      const float* w = p.ws + ((long long)z * p.splits * p.M) * p.N;
      for (int e = threadIdx.x; e < mt * W_TILE; e += GEMM_THREADS) {
        const int ml = e / W_TILE, nl = e % W_TILE;
        if (nl >= nt) continue;
        float acc = 0.0f;
        for (int s = 0; s < p.splits; ++s) acc += w[((long long)s * p.M + m0 + ml) * p.N + n0 + nl];
        p.C[z * p.c_bs + (long long)(m0 + ml) * p.ldc + n0 + nl] = f2bf(acc);
      }
    }
  }

  tc::tc_fence_before();
  __syncthreads();
  if (*abort_flag) {
    // a wait was given up: let copies and MMAs in flight settle before TMEM is released
    for (int i = 0; i < 2000; ++i) __nanosleep(1000);
  }
  if (warp == 1) {
    tc::tc_fence_after();
    tc::tmem_dealloc(tmem, TMEM_COLS);
  }
}

struct Workspace {
  float* ws = nullptr;
  size_t ws_elems = 0;
  unsigned* counters = nullptr;
  size_t n_counters = 0;
};
Workspace g_ws[64];  // per device

int pick_nt(int M) { return M <= 16 ? 16 : M <= 32 ? 32 : M <= 64 ? 64 : M <= 128 ? 128 : 256; }

}  // namespace

bool gemm_tc_supported(const GemmArgs& g) {
  if (g.b_kn || g.M <= 0 || g.N <= 0 || g.K <= 0) return false;
  if (g.K % 8 || g.lda % 8 || g.ldb % 8 || g.a_bs % 8 || g.b_bs % 8) return false;
  if ((reinterpret_cast<uintptr_t>(g.A) & 15) || (reinterpret_cast<uintptr_t>(g.B) & 15)) return false;
  return true;
}

cudaError_t launch_gemm_tc(const GemmArgs& g, int* d_status, cudaStream_t st) {
  int dev = 0, n_sm = 0;
  cudaError_t e = cudaGetDevice(&dev);
  if (e != cudaSuccess) return e;
  cudaDeviceGetAttribute(&n_sm, cudaDevAttrMultiProcessorCount, dev);
  const int NT = pick_nt(g.M);
  const int n_tiles = (g.N + W_TILE - 1) / W_TILE, m_tiles = (g.M + NT - 1) / NT;
  const int kc_total = (g.K + BK - 1) / BK;
  // split K until the grid covers the SMs, keeping at least 4 K chunks per CTA
  int splits = 1;
  const long long tiles = (long long)n_tiles * m_tiles * g.batch;
  if (tiles < n_sm) splits = (int)std::min<long long>((n_sm + tiles - 1) / tiles, std::max(1, kc_total / 4));
  while (splits > 1 && (size_t)g.batch * splits * g.M * g.N > (size_t)(64u << 20)) --splits;

  Workspace& W = g_ws[dev & 63];
  const size_t need_ws = splits > 1 ? (size_t)g.batch * splits * g.M * g.N : 0;
  const size_t need_ctr = (size_t)tiles;
  if (need_ws > W.ws_elems) {
    if (W.ws) cudaFree(W.ws);
    W.ws = nullptr;
    W.ws_elems = 0;
    if ((e = cudaMalloc((void**)&W.ws, need_ws * sizeof(float))) != cudaSuccess) return e;
    W.ws_elems = need_ws;
  }
  if (need_ctr > W.n_counters) {
    if (W.counters) cudaFree(W.counters);
    W.counters = nullptr;
    W.n_counters = 0;
    const size_t n = std::max<size_t>(need_ctr, 4096);
    if ((e = cudaMalloc((void**)&W.counters, n * sizeof(unsigned))) != cudaSuccess) return e;
    if ((e = cudaMemset(W.counters, 0, n * sizeof(unsigned))) != cudaSuccess) return e;
    W.n_counters = n;
  }

  CUtensorMap tmW, tmA;
  const char* err = nullptr;
  // dimension order {K, rows, batch}, or {K, batch, rows} when the batch stride is the smaller
  // one, so that the byte strides of the map ascend
  auto build = [&](CUtensorMap* out, const bf16* base, int rows, int ld, long long bs, int box_rows, int* swap) {
    const uint64_t row_b = (uint64_t)ld * 2;
    const uint64_t bat_b = g.batch > 1 ? (uint64_t)bs * 2 : row_b * (uint64_t)rows;
    *swap = g.batch > 1 && bat_b < row_b;
    if (*swap)
      return tc::cached_tmap(out, base, g.K, g.batch, rows, bat_b, row_b, BK, 1, box_rows, &err);
    return tc::cached_tmap(out, base, g.K, rows, g.batch, row_b, std::max<uint64_t>(bat_b, 16), BK, box_rows, 1, &err);
  };
  int w_swap = 0, a_swap = 0;
  if (!build(&tmW, g.B, g.N, g.ldb, g.b_bs, W_TILE, &w_swap) || !build(&tmA, g.A, g.M, g.lda, g.a_bs, NT, &a_swap))
    return cudaErrorInvalidValue;

  GemmTcParams p;
  p.C = g.C; p.ws = W.ws; p.counters = W.counters; p.d_status = d_status;
  p.M = g.M; p.N = g.N; p.K = g.K; p.ldc = g.ldc; p.c_bs = g.c_bs;
  p.splits = splits; p.kc_total = kc_total; p.w_swap = w_swap; p.a_swap = a_swap;
  const int stage_bytes = W_BYTES + NT * BK * 2;
  p.stages = std::max(2, std::min(8, (200 * 1024) / stage_bytes));
  const size_t smem = (size_t)p.stages * stage_bytes + 1024 /* alignment */ + 256 /* barriers */;
  dim3 grid(n_tiles, m_tiles * splits, g.batch);

#define FST_LAUNCH_GEMM(NTV)                                                                      \
  do {                                                                                            \
    static bool attr_set = false;                                                                 \
    if (!attr_set) {                                                                              \
      e = cudaFuncSetAttribute(k_gemm_tc<NTV>, cudaFuncAttributeMaxDynamicSharedMemorySize, 227 * 1024); \
      if (e != cudaSuccess) return e;                                                             \
      attr_set = true;                                                                            \
    }                                                                                             \
    k_gemm_tc<NTV><<<grid, GEMM_THREADS, smem, st>>>(tmW, tmA, p);                                \
  } while (0)
  switch (NT) {
    case 16: FST_LAUNCH_GEMM(16); break;
    case 32: FST_LAUNCH_GEMM(32); break;
    case 64: FST_LAUNCH_GEMM(64); break;
    case 128: FST_LAUNCH_GEMM(128); break;
    default: FST_LAUNCH_GEMM(256); break;
  }
#undef FST_LAUNCH_GEMM
  return cudaGetLastError();
}

// ---- host: tensor map encoding through the driver entry point (no link-time libcuda) ----------
namespace tc {

typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                  const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                  CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

bool make_tmap_bf16(CUtensorMap* out, const void* base, int rank, const uint64_t* dims, const uint64_t* strides_bytes,
                    const uint32_t* box, const char** err) {
  static EncodeTiledFn fn = nullptr;
  if (!fn) {
    void* p = nullptr;
    cudaDriverEntryPointQueryResult q;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) != cudaSuccess || !p) {
      if (err) *err = "cuTensorMapEncodeTiled is not available";
      return false;
    }
    fn = reinterpret_cast<EncodeTiledFn>(p);
  }
  cuuint64_t gd[5];
  cuuint64_t gs[5];
  cuuint32_t bx[5], es[5];
  for (int i = 0; i < rank; ++i) {
    gd[i] = dims[i];
    bx[i] = box[i];
    es[i] = 1;
    if (i > 0) gs[i - 1] = strides_bytes[i - 1];
  }
  CUresult r = fn(out, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, (cuuint32_t)rank, const_cast<void*>(base), gd, gs, bx, es,
                  CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                  CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) {
    if (err) *err = "cuTensorMapEncodeTiled failed";
    return false;
  }
  return true;
}

namespace {
struct TmapKey {
  const void* base;
  uint64_t d0, d1, d2, s1, s2;
  uint32_t b0, b1, b2;
  bool operator==(const TmapKey& o) const {
    return base == o.base && d0 == o.d0 && d1 == o.d1 && d2 == o.d2 && s1 == o.s1 && s2 == o.s2 && b0 == o.b0 &&
           b1 == o.b1 && b2 == o.b2;
  }
};
struct TmapHash {
  size_t operator()(const TmapKey& k) const {
    size_t h = reinterpret_cast<size_t>(k.base);
    for (uint64_t v : {k.d0, k.d1, k.d2, k.s1, k.s2, (uint64_t)k.b0, (uint64_t)k.b1, (uint64_t)k.b2}) h = h * 1000003u ^ (size_t)v;
    return h;
  }
};

std::mutex g_mu;
std::unordered_map<TmapKey, CUtensorMap, TmapHash> g_tmaps;

}  // namespace

bool cached_tmap(CUtensorMap* out, const void* base, uint64_t d0, uint64_t d1, uint64_t d2, uint64_t s1,
                 uint64_t s2, uint32_t b0, uint32_t b1, uint32_t b2, const char** err) {
  TmapKey key{base, d0, d1, d2, s1, s2, b0, b1, b2};
  std::lock_guard<std::mutex> lk(g_mu);
  auto it = g_tmaps.find(key);
  if (it != g_tmaps.end()) {
    *out = it->second;
    return true;
  }
  const uint64_t dims[3] = {d0, d1, d2};
  const uint64_t strides[2] = {s1, s2};
  const uint32_t box[3] = {b0, b1, b2};
  if (!make_tmap_bf16(out, base, 3, dims, strides, box, err)) return false;
  if (g_tmaps.size() > 4096) g_tmaps.clear();
  g_tmaps.emplace(key, *out);
  return true;
}


}  // namespace tc
}  // namespace fst
