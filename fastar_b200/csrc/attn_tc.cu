// Split-KV latent attention on tcgen05 / TMEM / TMA: the QK, softmax and SV stages of
// process_mla (reference src/fst_engine.cpp:3573-3683) fused with an online softmax over the
// paged bf16 cache, for 64 heads sharing every cached row.
//
// Orientation.  With one query token the natural M dimension (64 heads) would leave half of a
// 128-row tcgen05.mma idle, so both products are transposed and the CACHED TOKENS are M:
//   S^T[128 tok, 64 heads] = K[128 tok, d_qk] * Q^T          (A = cache tile, K-major;
//                                                             B = Q_eff, K-major)
//   O^T[512, 64 heads]    += V^T[512, 128 tok] * P^T          (A = the same cache bytes read
//                                                             MN-major; B = P, MN-major)
// A cached row is fetched from HBM once and serves as key and as value.
//
// One persistent CTA per SM walks its run of schedule segments.  Shared memory holds Q_eff
// (64 x d_qk) and ONE 128-token tile as d_qk/64 chunks of [128 tok x 64 dims] in the 128-byte
// swizzle that TMA writes and UMMA reads.  Chunks are the unit of the pipeline: a chunk is
// refilled with the next tile's data as soon as the SV MMAs that read it have retired, and the
// QK MMAs of the next tile start on the chunks that have landed.  With 576-wide rows the
// rope chunk is dead after QK, so P^T is written over it.
//
// Warp roles: warp 0 lane 0 issues TMA; warp 1 lane 0 issues tcgen05.mma (warp 1 owns the TMEM
// allocation); warps 2-5 are the softmax / epilogue threads, one cached token (TMEM lane) each.
// TMEM: S^T in columns [0, 64), O^T in 4 x 64 columns from 64.
#include "kernels.cuh"
#include "tc_common.cuh"

namespace fst {

namespace {

constexpr int TILE = 128;        // cached tokens per tile (2 pages of 64)
constexpr int HEADS = 64;
constexpr int D_V = 512;
constexpr int Q_CHUNK = HEADS * 128;   // bytes of one [64 x 64] bf16 chunk of Q
constexpr int KV_CHUNK = TILE * 128;   // bytes of one [128 x 64] bf16 chunk of the tile
constexpr int ATTN_THREADS = 192;
constexpr uint32_t TMEM_COLS = 512;
constexpr uint32_t COL_S = 0, COL_O = 64;
constexpr float RESCALE_THRESHOLD = 8.0f;  // log2 units: O is rescaled only when the max grows by > 2^8

struct AttnTcParams {
  const int32_t* tables;
  const int32_t* tok_table;
  const AttnSeg* segs;
  const int32_t* cta_seg;
  float* part_m;
  float* part_l;
  float* part_o;
  int* d_status;
  int pool_rows;   // first row index outside the pool: TMA fills zeros there
  float scale_log2;
};

template <int NCH>
struct Smem {
  static constexpr int Q_BYTES = NCH * Q_CHUNK;
  static constexpr int KV_BYTES = NCH * KV_CHUNK;
  static constexpr bool P_IN_TILE = NCH == 9;  // 576-wide rows: P^T overwrites the rope chunk
  static constexpr int P_OFF = P_IN_TILE ? Q_BYTES + 8 * KV_CHUNK : Q_BYTES + KV_BYTES;
  static constexpr int MISC_OFF = Q_BYTES + KV_BYTES + (P_IN_TILE ? 0 : KV_CHUNK);
  static constexpr int MISC_BYTES = 4096;
  static constexpr int TOTAL = MISC_OFF + MISC_BYTES + 1024;
};

struct Misc {
  uint64_t q_full;
  uint64_t kv_full[9];
  uint64_t kv_empty[9];
  uint64_t s_full;
  uint64_t p_full;
  uint64_t o_done;
  uint32_t tmem_slot;
  int abort_flag;
  int rescale;
  int pad;
  float wmax[4][HEADS];   // per-warp tile maxima / per-warp row sums in the epilogue
  float m_used[HEADS];    // running reference maximum (log2 units), the same for all threads
  float alpha[HEADS];     // rescale factor of this tile
};

__device__ __forceinline__ float redux_max(float v) {
  float r;
  asm volatile("redux.sync.max.f32 %0, %1, 0xffffffff;" : "=f"(r) : "f"(v));
  return r;
}
__device__ __forceinline__ void softmax_bar() { asm volatile("bar.sync 1, 128;" ::: "memory"); }
// Barrier of the 128 softmax threads that also ANDs a flag, so that a wait given up by one
// warp ends the loop of all four and nobody is left waiting at a later barrier.
__device__ __forceinline__ bool softmax_bar_and(bool v) {
  uint32_t out;
  asm volatile(
      "{\n\t.reg .pred q, r;\n\t"
      "setp.ne.u32 q, %1, 0;\n\t"
      "bar.red.and.pred r, 1, 128, q;\n\t"
      "selp.u32 %0, 1, 0, r;\n\t}"
      : "=r"(out)
      : "r"((uint32_t)v)
      : "memory");
  return out != 0;
}

template <int NCH>
__global__ void __launch_bounds__(ATTN_THREADS, 1)
k_attn_tc(const __grid_constant__ CUtensorMap tmQ, const __grid_constant__ CUtensorMap tmKV, AttnTcParams p) {
  using L = Smem<NCH>;
  extern __shared__ __align__(1024) unsigned char smem_raw[];
  unsigned char* smem = reinterpret_cast<unsigned char*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  unsigned char* s_q = smem;
  unsigned char* s_kv = smem + L::Q_BYTES;
  unsigned char* s_p = smem + L::P_OFF;
  Misc* mi = reinterpret_cast<Misc*>(smem + L::MISC_OFF);
  volatile int* abort_flag = &mi->abort_flag;

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int seg0 = p.cta_seg[blockIdx.x], seg1 = p.cta_seg[blockIdx.x + 1];

  if (threadIdx.x == 0) {
    tc::mbar_init(&mi->q_full, 1);
    for (int c = 0; c < 9; ++c) {
      tc::mbar_init(&mi->kv_full[c], 1);
      tc::mbar_init(&mi->kv_empty[c], 1);
    }
    tc::mbar_init(&mi->s_full, 1);
    tc::mbar_init(&mi->p_full, 128);
    tc::mbar_init(&mi->o_done, 1);
    mi->abort_flag = 0;
    mi->rescale = 0;
    tc::fence_barrier_init();
  }
  if (warp == 1) tc::tmem_alloc(&mi->tmem_slot, TMEM_COLS);
  tc::tc_fence_before();
  __syncthreads();
  tc::tc_fence_after();
  const uint32_t tmem = mi->tmem_slot;

  if (warp == 0) {
    // ---------------- TMA producer ----------------
    if (lane == 0) {
      tc::tma_prefetch_desc(&tmQ);
      tc::tma_prefetch_desc(&tmKV);
      int g = 0;
      bool ok = true;
      for (int si = seg0; si < seg1 && ok; ++si) {
        const AttnSeg sg = p.segs[si];
        const int32_t* table = p.tables + p.tok_table[sg.tok];
        const int n_tiles = (sg.kv_end - sg.kv_begin + TILE - 1) / TILE;
        for (int t = 0; t < n_tiles && ok; ++t, ++g) {
          const int base = sg.kv_begin + t * TILE;
          const int row0 = table[base >> 6] * 64;
          const int row1 = base + 64 < sg.kv_end ? table[(base >> 6) + 1] * 64 : p.pool_rows;
          for (int c = 0; c < NCH; ++c) {
            if (g > 0) {
              ok = tc::mbar_wait(&mi->kv_empty[c], (g - 1) & 1, abort_flag, p.d_status, ST_TMA_TIMEOUT);
              if (!ok) break;
            }
            if (t == 0 && c == 0) {
              // the QK MMAs of the previous segment have retired (they precede the SV MMAs
              // that freed chunk 0), so Q_eff may be replaced
              tc::mbar_expect_tx(&mi->q_full, L::Q_BYTES);
              for (int cc = 0; cc < NCH; ++cc)
                tc::tma_load_3d(s_q + cc * Q_CHUNK, &tmQ, &mi->q_full, cc * 64, sg.tok * HEADS, 0);
            }
            tc::mbar_expect_tx(&mi->kv_full[c], KV_CHUNK);
            tc::tma_load_3d(s_kv + c * KV_CHUNK, &tmKV, &mi->kv_full[c], c * 64, row0, 0);
            tc::tma_load_3d(s_kv + c * KV_CHUNK + KV_CHUNK / 2, &tmKV, &mi->kv_full[c], c * 64, row1, 0);
          }
        }
      }
    }
  } else if (warp == 1) {
    // ---------------- MMA issuer ----------------
    if (lane == 0) {
      constexpr uint32_t idesc_qk = tc::umma_idesc_bf16(TILE, HEADS, 0, 0);
      constexpr uint32_t idesc_sv = tc::umma_idesc_bf16(128, HEADS, 1, 1);
      const uint32_t q_addr = tc::smem_u32(s_q), kv_addr = tc::smem_u32(s_kv), p_addr = tc::smem_u32(s_p);
      int g = 0, sidx = 0;
      bool ok = true;
      for (int si = seg0; si < seg1 && ok; ++si, ++sidx) {
        const AttnSeg sg = p.segs[si];
        const int n_tiles = (sg.kv_end - sg.kv_begin + TILE - 1) / TILE;
        ok = tc::mbar_wait(&mi->q_full, sidx & 1, abort_flag, p.d_status, ST_MMA_TIMEOUT);
        for (int t = 0; t < n_tiles && ok; ++t, ++g) {
          // S^T = K * Q^T, chunk by chunk as the tile lands
          for (int c = 0; c < NCH && ok; ++c) {
            ok = tc::mbar_wait(&mi->kv_full[c], g & 1, abort_flag, p.d_status, ST_MMA_TIMEOUT);
            if (!ok) break;
            tc::tc_fence_after();
#pragma unroll
            for (int k = 0; k < 4; ++k) {
              const uint64_t da = tc::umma_desc_sw128(kv_addr + c * KV_CHUNK + k * 32, 16, 1024);
              const uint64_t db = tc::umma_desc_sw128(q_addr + c * Q_CHUNK + k * 32, 16, 1024);
              tc::umma_bf16(tmem + COL_S, da, db, idesc_qk, (c > 0 || k > 0) ? 1u : 0u);
            }
          }
          if (!ok) break;
          tc::umma_commit(&mi->s_full);
          // O^T += V^T * P^T once the softmax threads have written P^T
          ok = tc::mbar_wait(&mi->p_full, g & 1, abort_flag, p.d_status, ST_MMA_TIMEOUT);
          if (!ok) break;
          tc::tc_fence_after();
#pragma unroll
          for (int mt = 0; mt < 4; ++mt) {
#pragma unroll
            for (int k = 0; k < TILE / 16; ++k) {
              // A: d rows 128*mt .. +127 (chunks 2mt, 2mt+1: LBO = chunk stride), tokens 16k .. +15
              const uint64_t da = tc::umma_desc_sw128(kv_addr + 2 * mt * KV_CHUNK + k * 2048, KV_CHUNK, 1024);
              const uint64_t db = tc::umma_desc_sw128(p_addr + k * 2048, 16, 1024);
              tc::umma_bf16(tmem + COL_O + mt * HEADS, da, db, idesc_sv, (t > 0 || k > 0) ? 1u : 0u);
            }
            tc::umma_commit(&mi->kv_empty[2 * mt]);
            tc::umma_commit(&mi->kv_empty[2 * mt + 1]);
          }
          if (NCH == 9) tc::umma_commit(&mi->kv_empty[8]);
          tc::umma_commit(&mi->o_done);
        }
      }
    }
  } else {
    // ---------------- softmax / epilogue: thread = one cached token of the tile ----------------
    const int quad = warp & 3;
    const int tok_in_tile = quad * 32 + lane;
    const uint32_t lane_addr = tmem + ((uint32_t)(quad * 32) << 16);
    const int sm_tid = threadIdx.x - 64;  // 0..127
    int g = 0;
    bool ok = true;
    for (int si = seg0; si < seg1 && ok; ++si) {
      const AttnSeg sg = p.segs[si];
      const int n_tiles = (sg.kv_end - sg.kv_begin + TILE - 1) / TILE;
      float l[HEADS];
#pragma unroll
      for (int h = 0; h < HEADS; ++h) l[h] = 0.0f;
      if (sm_tid < HEADS) mi->m_used[sm_tid] = -INFINITY;
      softmax_bar();
      for (int t = 0; t < n_tiles && ok; ++t, ++g) {
        ok = tc::mbar_wait(&mi->s_full, g & 1, abort_flag, p.d_status, ST_SOFTMAX_TIMEOUT);
        tc::tc_fence_after();
        const bool valid = sg.kv_begin + t * TILE + tok_in_tile < sg.kv_end;
        // pass 1: per-warp maxima over the warp's 32 tokens, for every head
#pragma unroll
        for (int half = 0; half < 2; ++half) {
          float s[32];
          tc::tmem_ld32(lane_addr + COL_S + half * 32, s);
#pragma unroll
          for (int j = 0; j < 32; ++j) {
            const float v = valid ? s[j] * p.scale_log2 : -INFINITY;
            const float r = redux_max(v);
            if (lane == j) mi->wmax[quad][half * 32 + j] = r;
          }
        }
        ok = softmax_bar_and(ok);
        if (!ok) break;
        // one thread per head decides whether the reference maximum moves
        if (sm_tid < HEADS) {
          const float tm = fmaxf(fmaxf(mi->wmax[0][sm_tid], mi->wmax[1][sm_tid]),
                                 fmaxf(mi->wmax[2][sm_tid], mi->wmax[3][sm_tid]));
          const float mo = mi->m_used[sm_tid];
          float a = 1.0f;
          if (tm > mo + RESCALE_THRESHOLD) {  // also the first tile (mo = -inf)
            a = exp2f(mo - tm);
            mi->m_used[sm_tid] = tm;
            if (t > 0) mi->rescale = 1;
          }
          mi->alpha[sm_tid] = a;
        }
        softmax_bar();
        const bool rescale = mi->rescale != 0;
        // pass 2: P = exp2(s - m), row sums, P^T into shared memory (MN-major, 128-byte swizzle)
#pragma unroll
        for (int half = 0; half < 2; ++half) {
          float s[32];
          tc::tmem_ld32(lane_addr + COL_S + half * 32, s);
          uint32_t packed[16];
#pragma unroll
          for (int j = 0; j < 32; j += 2) {
            const int h = half * 32 + j;
            const float p0 = valid ? exp2f(s[j] * p.scale_log2 - mi->m_used[h]) : 0.0f;
            const float p1 = valid ? exp2f(s[j + 1] * p.scale_log2 - mi->m_used[h + 1]) : 0.0f;
            if (rescale) {
              l[h] *= mi->alpha[h];
              l[h + 1] *= mi->alpha[h + 1];
            }
            l[h] += p0;
            l[h + 1] += p1;
            __nv_bfloat162 b = __floats2bfloat162_rn(p0, p1);
            packed[j / 2] = *reinterpret_cast<uint32_t*>(&b);
          }
          unsigned char* prow = s_p + tok_in_tile * 128;
#pragma unroll
          for (int q4 = 0; q4 < 4; ++q4) {
            const int chunk = (half * 4 + q4) ^ (tok_in_tile & 7);
            *reinterpret_cast<uint4*>(prow + chunk * 16) =
                make_uint4(packed[q4 * 4], packed[q4 * 4 + 1], packed[q4 * 4 + 2], packed[q4 * 4 + 3]);
          }
        }
        // the reference maximum moved: rescale O^T (thread = one row of each 128-row block).
        // s_full of this tile implies that the SV MMAs of the previous tile have retired.
        if (rescale) {
#pragma unroll 1
          for (int blk = 0; blk < 8; ++blk) {
            float o[32];
            const uint32_t addr = lane_addr + COL_O + blk * 32;
            tc::tmem_ld32(addr, o);
#pragma unroll
            for (int j = 0; j < 32; ++j) o[j] *= mi->alpha[(blk & 1) * 32 + j];
            tc::tmem_st32(addr, o);
          }
        }
        tc::fence_proxy_async();
        tc::tc_fence_before();
        softmax_bar();  // every thread has read alpha / rescale before they are reset
        if (sm_tid == 0) mi->rescale = 0;
        tc::mbar_arrive(&mi->p_full);
      }
      if (!ok) break;
      // ---- epilogue of the segment: un-normalised partial (max, sum, O) ----
      ok = tc::mbar_wait(&mi->o_done, (g - 1) & 1, abort_flag, p.d_status, ST_EPI_TIMEOUT);
      tc::tc_fence_after();
#pragma unroll
      for (int h = 0; h < HEADS; ++h) {
        const float v = warp_sum(l[h]);
        if (lane == (h & 31)) mi->wmax[quad][h] = v;
      }
      ok = softmax_bar_and(ok);
      if (!ok) break;
      if (sm_tid < HEADS) {
        const float sum = mi->wmax[0][sm_tid] + mi->wmax[1][sm_tid] + mi->wmax[2][sm_tid] + mi->wmax[3][sm_tid];
        p.part_l[(long long)sg.part * HEADS + sm_tid] = sum;
        p.part_m[(long long)sg.part * HEADS + sm_tid] = mi->m_used[sm_tid] * 0.6931471805599453f;  // back to ln units
      }
      float* po = p.part_o + (long long)sg.part * HEADS * D_V;
#pragma unroll 1
      for (int blk = 0; blk < 8; ++blk) {
        float o[32];
        tc::tmem_ld32(lane_addr + COL_O + blk * 32, o);
        const int d = (blk >> 1) * 128 + tok_in_tile;  // row of O^T
#pragma unroll
        for (int j = 0; j < 32; ++j) po[(long long)((blk & 1) * 32 + j) * D_V + d] = o[j];
      }
      tc::tc_fence_before();
      softmax_bar();  // wmax / m_used are reused by the next segment
    }
  }

  tc::tc_fence_before();
  __syncthreads();
  if (*abort_flag) {
    for (int i = 0; i < 2000; ++i) __nanosleep(1000);  // let copies and MMAs in flight settle
  }
  if (warp == 1) {
    tc::tc_fence_after();
    tc::tmem_dealloc(tmem, TMEM_COLS);
  }
}

}  // namespace

bool attn_tc_supported(const AttnArgs& a) {
  return a.H == HEADS && a.d_v == D_V && a.page_tokens == 64 && a.row == a.d_qk &&
         (a.d_qk == 576 || a.d_qk == 512) && a.pool_rows < (1ll << 31) &&
         (reinterpret_cast<uintptr_t>(a.pool) & 15) == 0 && (reinterpret_cast<uintptr_t>(a.q_eff) & 15) == 0;
}

size_t attn_tc_smem_bytes(const AttnArgs& a) { return a.d_qk == 576 ? Smem<9>::TOTAL : Smem<8>::TOTAL; }

cudaError_t launch_attn_tc(const AttnArgs& a, cudaStream_t st) {
  static_assert(sizeof(Misc) <= Smem<9>::MISC_BYTES, "misc region too small");
  static_assert(Smem<9>::TOTAL <= 227 * 1024 && Smem<8>::TOTAL <= 227 * 1024, "shared memory budget");
  if (a.n_segs <= 0) return cudaSuccess;
  CUtensorMap tmQ, tmKV;
  const char* err = nullptr;
  // Q_eff [q_rows, d_qk] and the pool [pool_rows, row]: boxes of 64 dims x 64 rows
  if (!tc::cached_tmap(&tmQ, a.q_eff, (uint64_t)a.d_qk, (uint64_t)a.q_rows, 1, (uint64_t)a.d_qk * 2,
                       (uint64_t)a.d_qk * 2 * (uint64_t)a.q_rows, 64, 64, 1, &err) ||
      !tc::cached_tmap(&tmKV, a.pool, (uint64_t)a.row, (uint64_t)a.pool_rows, 1, (uint64_t)a.row * 2,
                       (uint64_t)a.row * 2 * (uint64_t)a.pool_rows, 64, 64, 1, &err))
    return cudaErrorInvalidValue;
  AttnTcParams p;
  p.tables = a.tables; p.tok_table = a.tok_table; p.segs = a.segs; p.cta_seg = a.cta_seg;
  p.part_m = a.part_m; p.part_l = a.part_l; p.part_o = a.part_o; p.d_status = a.d_status;
  p.pool_rows = (int)a.pool_rows;
  p.scale_log2 = a.scale * 1.4426950408889634f;
  cudaError_t e;
  if (a.d_qk == 576) {
    static bool set9 = false;
    if (!set9) {
      e = cudaFuncSetAttribute(k_attn_tc<9>, cudaFuncAttributeMaxDynamicSharedMemorySize, Smem<9>::TOTAL);
      if (e != cudaSuccess) return e;
      set9 = true;
    }
    k_attn_tc<9><<<a.n_ctas, ATTN_THREADS, Smem<9>::TOTAL, st>>>(tmQ, tmKV, p);
  } else {
    static bool set8 = false;
    if (!set8) {
      e = cudaFuncSetAttribute(k_attn_tc<8>, cudaFuncAttributeMaxDynamicSharedMemorySize, Smem<8>::TOTAL);
      if (e != cudaSuccess) return e;
      set8 = true;
    }
    k_attn_tc<8><<<a.n_ctas, ATTN_THREADS, Smem<8>::TOTAL, st>>>(tmQ, tmKV, p);
  }
  return cudaGetLastError();
}

}  // namespace fst
