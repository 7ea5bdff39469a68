// Skinny bf16 GEMM on the 5th-generation tensor cores: C[M, N] = A[M, K] * W^T with the weight
// rows as the MMA M dimension (128 per CTA) and the tokens as the MMA N dimension, so a handful
// of tokens still fills a 128-row tcgen05.mma.  This is the tile engine the reference calls
// npu_gemm_mla_vec (src/fst_engine.cpp:465-575): weights stay in their native layout -- [N, K]
// (the b_col_maj kernels) or [K, N] (the b_row_maj kernel, 480) -- and are streamed from HBM
// exactly once.
//
// One CTA = one (128-row weight tile, token tile, K slice).  Warp 0 streams both operands with
// TMA through a ring of 128-byte-swizzled stages; one lane of warp 1 issues tcgen05.mma into a
// TMEM accumulator; warps 2-5 drain TMEM.  The K slices of one output tile form a thread-block
// cluster: every CTA parks its fp32 partial in its own shared memory and then reduces one
// column slice of the tile over all peers through distributed shared memory, in rank order
// (deterministic), without a round trip through global memory.
#include <algorithm>
#include <mutex>
#include <unordered_map>

#include "kernels.cuh"
#include "tc_common.cuh"

namespace fst {

namespace {

constexpr int BK = 64;       // K elements per stage: one 128-byte swizzle span
constexpr int W_TILE = 128;  // weight rows per CTA
constexpr int W_BYTES = W_TILE * BK * 2;
constexpr int GEMM_THREADS = 192;
constexpr int MAX_SPLITS = 8;  // portable cluster size

struct GemmTcParams {
  bf16* C;
  int* d_status;
  int M, N, K, ldc;
  long long c_bs;
  int splits, kc_total, stages;
  int w_swap, a_swap;  // the batch index is the middle tensor-map coordinate (its stride is the smaller one)
  // side job (GemmArgs::rope_*): null source = none
  const bf16* rope_src;
  const float* rope_lut;
  bf16* rope_dst;
  int rope_T, rope_H, rope_q_head, rope_nope, rope_dims, rope_d_qk;
  const int* status_dev;  // GemmArgs::status_dev / status_host
  int* status_host;
};

__device__ __forceinline__ uint32_t cluster_ctarank() {
  uint32_t r;
  asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
  return r;
}
__device__ __forceinline__ void cluster_sync_all() {
  asm volatile("barrier.cluster.arrive.release.aligned;\n\tbarrier.cluster.wait.acquire.aligned;" ::: "memory");
}
// 16 bytes from the same shared-memory offset of the cluster's CTA `rank`.
__device__ __forceinline__ float4 ld_peer_f32x4(uint32_t local_addr, uint32_t rank) {
  uint32_t remote;
  float4 v;
  asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(remote) : "r"(local_addr), "r"(rank));
  asm volatile("ld.shared::cluster.v4.f32 {%0, %1, %2, %3}, [%4];"
               : "=f"(v.x), "=f"(v.y), "=f"(v.z), "=f"(v.w)
               : "r"(remote)
               : "memory");
  return v;
}

// NT: token tile (MMA N).  W_KN: the weight operand is stored [K, N] (N contiguous) and is read
// as an MN-major UMMA operand; otherwise [N, K], K-major.
template <int NT, bool W_KN>
__global__ void __launch_bounds__(GEMM_THREADS, 2)
k_gemm_tc(const __grid_constant__ CUtensorMap tmW, const __grid_constant__ CUtensorMap tmA, GemmTcParams p) {
  extern __shared__ __align__(1024) unsigned char smem_raw[];
  constexpr int A_BYTES = NT * BK * 2;
  constexpr int STAGE_BYTES = W_BYTES + A_BYTES;
  constexpr uint32_t TMEM_COLS = NT < 32 ? 32 : NT;
  constexpr int RED_BYTES = NT * W_TILE * 4;  // fp32 partial tile, parked over the ring
  unsigned char* smem = reinterpret_cast<unsigned char*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  const int ring = p.stages * STAGE_BYTES;
  unsigned char* misc = smem + ((p.splits == 1 || ring > RED_BYTES) ? ring : RED_BYTES);
  uint64_t* full = reinterpret_cast<uint64_t*>(misc);
  uint64_t* empty = full + 8;
  uint64_t* acc_bar = empty + 8;
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(acc_bar + 1);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

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
      auto load_w = [&](int i) {
        const int s = i % p.stages;
        unsigned char* st = smem + (size_t)s * STAGE_BYTES;
        const int k0 = (kc0 + i) * BK;
        tc::mbar_expect_tx(&full[s], STAGE_BYTES);
        if (W_KN) {
          // two boxes of [64 k rows x 64 n]: n is the innermost coordinate
          tc::tma_load_3d(st, &tmW, &full[s], n0, k0, z);
          tc::tma_load_3d(st + W_BYTES / 2, &tmW, &full[s], n0 + 64, k0, z);
        } else {
          tc::tma_load_3d(st, &tmW, &full[s], k0, p.w_swap ? z : n0, p.w_swap ? n0 : z);
        }
      };
      auto load_a = [&](int i) {
        const int s = i % p.stages;
        tc::tma_load_3d(smem + (size_t)s * STAGE_BYTES + W_BYTES, &tmA, &full[s], (kc0 + i) * BK, p.a_swap ? z : m0,
                        p.a_swap ? m0 : z);
      };
      // Weights are written by no kernel: the first ring of weight tiles is requested while the
      // previous kernel still runs; the activations are its output and wait for it.
      const int first = min(n_kc, p.stages);
      for (int i = 0; i < first; ++i) load_w(i);
      pdl_launch();
      pdl_wait();
      for (int i = 0; i < first; ++i) load_a(i);
      for (int i = first; i < n_kc; ++i) {
        if (!tc::mbar_wait(&empty[i % p.stages], ((i / p.stages) - 1) & 1, abort_flag, p.d_status, ST_TMA_TIMEOUT)) break;
        load_w(i);
        load_a(i);
      }
    } else {
      pdl_wait();
    }
  } else if (warp == 1) {
    pdl_wait();
    if (lane == 0) {
      constexpr uint32_t idesc = tc::umma_idesc_bf16(W_TILE, NT, W_KN ? 1 : 0, 0);
      // descriptors differ only in the start-address field: keep the rest in registers
      const uint64_t w_tmpl = W_KN ? tc::umma_desc_sw128(0, W_BYTES / 2, 1024) : tc::umma_desc_sw128(0, 16, 1024);
      const uint64_t a_tmpl = tc::umma_desc_sw128(0, 16, 1024);
      // 14-bit start-address field: inside a cluster the shared-window address of a CTA carries
      // its rank in high bits, which must not leak into the neighbouring descriptor fields
      const uint32_t base = tc::smem_u32(smem) & 0x3FFFFu;
      bool ok = true;
      for (int i = 0; i < n_kc && ok; ++i) {
        const int s = i % p.stages;
        ok = tc::mbar_wait(&full[s], (i / p.stages) & 1, abort_flag, p.d_status, ST_MMA_TIMEOUT);
        if (!ok) break;
        tc::tc_fence_after();
        const uint32_t w16 = (base + s * STAGE_BYTES) >> 4, a16 = w16 + (W_BYTES >> 4);
#pragma unroll
        for (int k = 0; k < BK / 16; ++k) {
          // K-major: 16 k = 32 bytes along the row; MN-major: 16 k rows of 128 bytes
          const uint64_t da = w_tmpl | (uint64_t)(w16 + (W_KN ? k * 128 : k * 2));
          const uint64_t db = a_tmpl | (uint64_t)(a16 + k * 2);
          tc::umma_bf16(tmem, da, db, idesc, (i > 0 || k > 0) ? 1u : 0u);
        }
        tc::umma_commit(&empty[s]);  // the stage is free once these MMAs have read it
      }
      if (ok) tc::umma_commit(acc_bar);
    }
  } else {
    // epilogue warps: TMEM lane quadrant = warp % 4; thread = one weight row n
    pdl_wait();
    // side job while the accumulator is being built: RoPE of head z's rope pairs.  Few tokens: the
    // head's first block takes them all (spreading them bought nothing at 64 tokens); many tokens
    // (verify blocks, prefill): every block of the head takes a slice, or the one block's 16 rounds
    // of dependent loads outlast the whole GEMM.
    const int rope_blocks = p.rope_T > 128 ? (int)(gridDim.x * gridDim.y) : 1;
    const int rope_id = (int)(blockIdx.y * gridDim.x + blockIdx.x);
    if (p.rope_src && rope_id < rope_blocks) {
      const int half = p.rope_dims / 2, et = threadIdx.x - 64;  // 128 epilogue threads
      const int t_lo = (int)((long long)p.rope_T * rope_id / rope_blocks), t_hi = (int)((long long)p.rope_T * (rope_id + 1) / rope_blocks);
      const int n_items = t_hi * half;
      for (int i0 = t_lo * half + et; i0 < n_items; i0 += 8 * (GEMM_THREADS - 64)) {
        // eight items per thread and round, all loads before the first store
        __nv_bfloat162 x[8];
        float2 cs[8];
#pragma unroll
        for (int u = 0; u < 8; ++u) {
          const int i = i0 + u * (GEMM_THREADS - 64);
          if (i < n_items) {
            const int t = i / half, pr = i % half;
            x[u] = *reinterpret_cast<const __nv_bfloat162*>(p.rope_src + ((long long)t * p.rope_H + z) * p.rope_q_head + p.rope_nope + 2 * pr);
            cs[u] = *reinterpret_cast<const float2*>(p.rope_lut + (long long)t * p.rope_dims + 2 * pr);
          }
        }
#pragma unroll
        for (int u = 0; u < 8; ++u) {
          const int i = i0 + u * (GEMM_THREADS - 64);
          if (i < n_items) {
            const int t = i / half, pr = i % half;
            const float x0 = __low2float(x[u]), x1 = __high2float(x[u]);
            *reinterpret_cast<__nv_bfloat162*>(p.rope_dst + ((long long)t * p.rope_H + z) * p.rope_d_qk + p.rope_d_qk - p.rope_dims + 2 * pr) =
                __floats2bfloat162_rn(x0 * cs[u].x - x1 * cs[u].y, x0 * cs[u].y + x1 * cs[u].x);
          }
        }
      }
    }
    const int quad = warp & 3;
    bool ok = n_kc == 0 || tc::mbar_wait(acc_bar, 0, abort_flag, p.d_status, ST_EPI_TIMEOUT);
    ok = __all_sync(0xffffffffu, ok);  // the TMEM loads below are warp-collective
    tc::tc_fence_after();
    const int row = quad * 32 + lane;
    const int n = n0 + row;
    // whether this block's output rows can go out as 8-byte stores (four weight rows per store)
    const bool wide_out = p.splits == 1 && (p.ldc % 4) == 0 && (p.c_bs % 4) == 0 && (n0 % 4) == 0 && n0 + W_TILE <= p.N &&
                          (reinterpret_cast<uintptr_t>(p.C) & 7) == 0;
    if (wide_out) {
      // the four epilogue warps take the staged path together or not at all (a wait that one of
      // them gave up must not leave the others at the barriers below)
      uint32_t all_ok;
      asm volatile(
          "{\n\t.reg .pred q, r;\n\t"
          "setp.ne.u32 q, %1, 0;\n\t"
          "bar.red.and.pred r, 1, 128, q;\n\t"
          "selp.u32 %0, 1, 0, r;\n\t}"
          : "=r"(all_ok)
          : "r"((uint32_t)ok)
          : "memory");
      ok = all_ok != 0;
    }
    if (ok && wide_out) {
      // No K split: the tile leaves through shared memory (the ring is idle once acc_bar fired), 32
      // tokens at a time, so that a warp writes 256 contiguous bytes of one token's row instead of
      // every thread two bytes per token.
      float* red = reinterpret_cast<float*>(smem);  // [32][128]
      const int e = threadIdx.x - 64;
      for (int c0 = 0; c0 < NT; c0 += 32) {
        if (m0 + c0 >= p.M) break;
        float v[32];
        if (n_kc > 0) {
          tc::tmem_ld32(tmem + ((uint32_t)(quad * 32) << 16) + c0, v);
        } else {
#pragma unroll
          for (int j = 0; j < 32; ++j) v[j] = 0.0f;
        }
#pragma unroll
        for (int j = 0; j < 32; ++j)
          if (j < NT - c0) red[j * W_TILE + row] = v[j];
        asm volatile("bar.sync 1, 128;" ::: "memory");
        const int n_tok = min(min(32, NT - c0), p.M - m0 - c0);
        for (int idx = e; idx < n_tok * (W_TILE / 4); idx += GEMM_THREADS - 64) {
          const int tok = idx / (W_TILE / 4), r4 = (idx % (W_TILE / 4)) * 4;
          const float4 f = *reinterpret_cast<const float4*>(red + tok * W_TILE + r4);
          const __nv_bfloat162 lo = __floats2bfloat162_rn(f.x, f.y), hi = __floats2bfloat162_rn(f.z, f.w);
          *reinterpret_cast<uint2*>(p.C + z * p.c_bs + (long long)(m0 + c0 + tok) * p.ldc + n0 + r4) =
              make_uint2(*reinterpret_cast<const uint32_t*>(&lo), *reinterpret_cast<const uint32_t*>(&hi));
        }
        asm volatile("bar.sync 1, 128;" ::: "memory");
      }
    } else if (ok) {
      float* red = reinterpret_cast<float*>(smem);  // [NT][128]: the ring is idle once acc_bar fired
      for (int c0 = 0; c0 < NT; c0 += 32) {
        if (p.splits == 1 && m0 + c0 >= p.M) break;
        float v[32];
        if (n_kc > 0) {
          tc::tmem_ld32(tmem + ((uint32_t)(quad * 32) << 16) + c0, v);
        } else {
#pragma unroll
          for (int j = 0; j < 32; ++j) v[j] = 0.0f;
        }
        if (p.splits == 1) {
          if (n < p.N) {
            bf16* c = p.C + z * p.c_bs + n;
#pragma unroll
            for (int j = 0; j < 32; ++j)
              if (j < NT - c0 && m0 + c0 + j < p.M) c[(long long)(m0 + c0 + j) * p.ldc] = f2bf(v[j]);
          }
        } else {
#pragma unroll
          for (int j = 0; j < 32; ++j)
            if (j < NT - c0) red[(c0 + j) * W_TILE + row] = v[j];
        }
      }
    }
  }

  __syncwarp();  // the single-lane roles rejoin their warps before the aligned barriers below
  if (p.splits > 1) {
    // every K slice has parked its partial: reduce one column slice of the tile over the
    // cluster, peers in rank order
    cluster_sync_all();
    const uint32_t rank = cluster_ctarank();
    const int c_lo = (int)(NT * rank / p.splits), c_hi = (int)(NT * (rank + 1) / p.splits);
    const uint32_t red_addr = tc::smem_u32(smem);
    for (int e4 = c_lo * (W_TILE / 4) + threadIdx.x; e4 < c_hi * (W_TILE / 4); e4 += GEMM_THREADS) {
      const int col = e4 / (W_TILE / 4), row = (e4 % (W_TILE / 4)) * 4;
      float4 v[MAX_SPLITS];
#pragma unroll
      for (int s = 0; s < MAX_SPLITS; ++s)  // all loads in flight before the first add
        v[s] = s < p.splits ? ld_peer_f32x4(red_addr + (uint32_t)e4 * 16, (uint32_t)s) : make_float4(0.f, 0.f, 0.f, 0.f);
      float acc[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
      for (int s = 0; s < MAX_SPLITS; ++s) {
        acc[0] += v[s].x;
        acc[1] += v[s].y;
        acc[2] += v[s].z;
        acc[3] += v[s].w;
      }
      if (m0 + col < p.M) {
        bf16* c = p.C + z * p.c_bs + (long long)(m0 + col) * p.ldc + n0 + row;
        if (n0 + row + 3 < p.N && (reinterpret_cast<uintptr_t>(c) & 7) == 0) {
          // one 8-byte store (the output may be page-locked host memory: fewer, fuller writes)
          const __nv_bfloat162 lo = __floats2bfloat162_rn(acc[0], acc[1]), hi = __floats2bfloat162_rn(acc[2], acc[3]);
          *reinterpret_cast<uint2*>(c) = make_uint2(*reinterpret_cast<const uint32_t*>(&lo), *reinterpret_cast<const uint32_t*>(&hi));
        } else {
#pragma unroll
          for (int j = 0; j < 4; ++j)
            if (n0 + row + j < p.N) c[j] = f2bf(acc[j]);
        }
      }
    }
    cluster_sync_all();  // nobody leaves while a peer still reads its shared memory
  }

  tc::tc_fence_before();
  __syncthreads();
  if (p.status_host && threadIdx.x == 0) {
    // (after this block's own waits: whatever it recorded itself is in the word it reads)
    const int st = *reinterpret_cast<const volatile int*>(p.status_dev);
    if (st != 0) *reinterpret_cast<volatile int*>(p.status_host) = st;
  }
  if (*abort_flag) {
    // a wait was given up: let copies and MMAs in flight settle before TMEM is released
    for (int i = 0; i < 2000; ++i) __nanosleep(1000);
  }
  if (warp == 1) {
    tc::tc_fence_after();
    tc::tmem_dealloc(tmem, TMEM_COLS);
  }
}

int pick_nt(int M) { return M <= 16 ? 16 : M <= 32 ? 32 : M <= 64 ? 64 : M <= 128 ? 128 : 256; }

template <int NT, bool W_KN>
cudaError_t launch_one(const CUtensorMap& tmW, const CUtensorMap& tmA, const GemmTcParams& p, dim3 grid, size_t smem,
                       cudaStream_t st) {
  return launch_pdl(k_gemm_tc<NT, W_KN>, grid, dim3(GEMM_THREADS, 1, 1), smem, st, p.splits, tmW, tmA, p);
}

}  // namespace

bool gemm_tc_supported(const GemmArgs& g) {
  if (g.M <= 0 || g.N <= 0 || g.K <= 0) return false;
  if (g.K % 8 || g.lda % 8 || g.ldb % 8 || g.a_bs % 8 || g.b_bs % 8) return false;
  if ((reinterpret_cast<uintptr_t>(g.A) & 15) || (reinterpret_cast<uintptr_t>(g.B) & 15)) return false;
  if (g.b_kn && g.N % 8) return false;
  return true;
}

cudaError_t launch_gemm_tc(const GemmArgs& g, int* d_status, cudaStream_t st) {
  int dev = 0, n_sm = 0;
  cudaError_t e = cudaGetDevice(&dev);
  if (e != cudaSuccess) return e;
  static int sm_count[64] = {0};
  if (!sm_count[dev & 63]) cudaDeviceGetAttribute(&sm_count[dev & 63], cudaDevAttrMultiProcessorCount, dev);
  n_sm = sm_count[dev & 63];
  int NT = pick_nt(g.M);
  const int n_tiles = (g.N + W_TILE - 1) / W_TILE;
  // a 256-token tile leaves no room for the parked partial: use it only when no K split is needed
  if (NT == 256 && (long long)n_tiles * ((g.M + 255) / 256) * g.batch * 2 <= 2ll * n_sm) NT = 128;
  const int m_tiles = (g.M + NT - 1) / NT;
  const int kc_total = (g.K + BK - 1) / BK;
  // K slices (a power of two, one cluster) while two CTAs per SM are not yet covered, keeping
  // at least two K chunks per CTA
  const long long tiles = (long long)n_tiles * m_tiles * g.batch;
  int splits = 1;
  while (splits < MAX_SPLITS && tiles * splits * 2 <= 2ll * n_sm && kc_total / (splits * 2) >= 2) splits *= 2;
  // Output tiles that cover half of the SMs or more are not split at all: a block per SM with a ring
  // of eight stages and no cluster reduction beats two half-size blocks on a third of the SMs
  // (the q-expand GEMM, 96 tiles: 18.2 -> 16.5 us; cut in three or four it was slower still).
  // With a handful of tokens the split wins (one token: 14.5 against 16.3 us).
  if (NT >= 64 && tiles * 2 >= n_sm && tiles <= n_sm) splits = 1;

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
  bool ok;
  if (g.b_kn) {
    // W is [K, N]: dims {N, K, batch}, boxes of 64 n x 64 k
    const uint64_t row_b = (uint64_t)g.ldb * 2;
    const uint64_t bat_b = g.batch > 1 ? (uint64_t)g.b_bs * 2 : row_b * (uint64_t)g.K;
    ok = tc::cached_tmap(&tmW, g.B, g.N, g.K, g.batch, row_b, std::max<uint64_t>(bat_b, 16), 64, BK, 1, &err);
  } else {
    ok = build(&tmW, g.B, g.N, g.ldb, g.b_bs, W_TILE, &w_swap);
  }
  if (!ok || !build(&tmA, g.A, g.M, g.lda, g.a_bs, NT, &a_swap)) return cudaErrorInvalidValue;

  GemmTcParams p;
  p.C = g.C; p.d_status = d_status;
  p.M = g.M; p.N = g.N; p.K = g.K; p.ldc = g.ldc; p.c_bs = g.c_bs;
  p.splits = splits; p.kc_total = kc_total; p.w_swap = w_swap; p.a_swap = a_swap;
  p.rope_src = g.rope_src; p.rope_lut = g.rope_lut; p.rope_dst = g.rope_dst;
  p.rope_T = g.rope_T; p.rope_H = g.rope_H; p.rope_q_head = g.rope_q_head; p.rope_nope = g.rope_nope;
  p.rope_dims = g.rope_dims; p.rope_d_qk = g.rope_d_qk;
  p.status_dev = g.status_host ? g.status_dev : nullptr; p.status_host = g.status_dev ? g.status_host : nullptr;
  const int stage_bytes = W_BYTES + NT * BK * 2;
  // Two blocks share an SM (96 KB of operand ring each) -- unless the grid has no more blocks than
  // there are SMs: then a block has the SM to itself anyway and takes a ring that holds its whole K
  // slice, so that every operand tile is requested at once instead of in two or three turns.
  const bool alone = tiles * splits <= n_sm;
  const int per_block = (kc_total + splits - 1) / splits;
  p.stages = std::max(2, std::min(std::min(8, alone ? per_block : 8), ((alone ? 192 : 96) * 1024) / stage_bytes));
  const size_t ring = (size_t)p.stages * stage_bytes, red = splits > 1 ? (size_t)NT * W_TILE * 4 : 0;
  const size_t smem = std::max(ring, red) + 1024 /* alignment */ + 256 /* barriers */;
  dim3 grid(n_tiles, m_tiles * splits, g.batch);

#define FST_GEMM_CASE(NTV)                                                                   \
  case NTV:                                                                                  \
    e = g.b_kn ? launch_one<NTV, true>(tmW, tmA, p, grid, smem, st)                          \
               : launch_one<NTV, false>(tmW, tmA, p, grid, smem, st);                        \
    break
  switch (NT) {
    FST_GEMM_CASE(16);
    FST_GEMM_CASE(32);
    FST_GEMM_CASE(64);
    FST_GEMM_CASE(128);
    default:
      e = g.b_kn ? launch_one<256, true>(tmW, tmA, p, grid, smem, st) : launch_one<256, false>(tmW, tmA, p, grid, smem, st);
      break;
  }
#undef FST_GEMM_CASE
  return e;
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
