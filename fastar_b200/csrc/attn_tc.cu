// Split-KV latent attention on tcgen05 / TMEM / TMA: the QK, softmax and SV stages of
// process_mla (reference src/fst_engine.cpp:3573-3683) fused with an online softmax over the
// paged bf16 cache, for 64 heads sharing every cached row.
//
// Orientation.  The score product is transposed so that the CACHED TOKENS are the MMA M
// dimension (a 128-row tcgen05.mma even with one query token), the value product is not, so
// that its N dimension is 256 latent columns wide:
//   S^T[128 tok, 64 heads] = K[128 tok, d_qk] * Q^T    (A = cache tile, K-major; B = Q_eff, K-major)
//   O[64 heads, 512]      += P[64 heads, 128 tok] * V  (A = P^T as written by the softmax threads,
//                                                       read MN-major; B = the same cache bytes,
//                                                       read MN-major, two halves of 256 columns)
// A cached row is fetched from HBM once and serves as key and as value.
//
// One persistent CTA per SM walks its run of schedule segments.  Shared memory holds Q_eff
// (64 x d_qk) and ONE 128-token tile as d_qk/64 chunks of [128 tok x 64 dims] in the 128-byte
// swizzle that TMA writes and UMMA reads.  Chunks are the unit of the pipeline: a chunk is
// refilled with the next tile's data as soon as the SV MMAs that read it have retired, and the
// QK MMAs of the next tile start on the chunks that have landed.  With 576-wide rows the
// rope chunk is dead after QK, so P^T is written over it.
//
// Warp roles: one lane of warps 0, 10 and 11 issues TMA (and prefetches the next tile into L2,
// so that the refill of a freed chunk is an L2 hit); warp 1 lane 0 issues tcgen05.mma (warp 1 owns the TMEM
// allocation); warps 2-9 are the softmax / epilogue threads: two per cached token (TMEM lane),
// 32 heads each.  TMEM: S^T in columns [0, 64).  O is two 64-row accumulators [64, 256] in
// columns [64, 320): a 64-row accumulator occupies lanes 0-15 of each 32-lane quadrant (head h
// in lane 32*(h/16) + h%16), so the second one sits at lane offset 16 in the same columns.
#include "kernels.cuh"
#include "tc_common.cuh"

namespace fst {

namespace {

constexpr int TILE = 128;        // cached tokens per tile (2 pages of 64)
constexpr int HEADS = 64;
constexpr int D_V = 512;
constexpr int Q_CHUNK = HEADS * 128;   // bytes of one [64 x 64] bf16 chunk of Q
constexpr int KV_CHUNK = TILE * 128;   // bytes of one [128 x 64] bf16 chunk of the tile
constexpr int ATTN_THREADS = 384;
constexpr int SOFTMAX_THREADS = 256;
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
  const bf16* pool;
  int pool_rows;   // first row index outside the pool: TMA fills zeros there
  float scale_log2;
};

#ifndef FST_PREFETCH
#define FST_PREFETCH 1
#endif
#ifndef FST_STAGGER
#define FST_STAGGER 1200
#endif
#ifdef FST_ATTN_TRACE
// Phase timestamps (SM clock) of CTA 0, for tuning builds only: [tile][event].
__device__ long long g_attn_trace[64 * 16];
#define TRACE(tile, ev) do { if (blockIdx.x == 0 && (tile) < 64) g_attn_trace[(tile) * 16 + (ev)] = clock64(); } while (0)
// Per-CTA summary: [cta][0..7] = global ns at entry, after the dependency wait, at exit; segments; SM clock at entry, exit.
__device__ long long g_attn_cta[256 * 8];
__device__ __forceinline__ long long gtime() { long long t; asm volatile("mov.u64 %0, %globaltimer;" : "=l"(t) : : "memory"); return t; }
#define CTA_TRACE(ev, val) do { if (threadIdx.x == 0 && blockIdx.x < 256) g_attn_cta[blockIdx.x * 8 + (ev)] = (val); } while (0)
#else
#define TRACE(tile, ev) do { } while (0)
#define CTA_TRACE(ev, val) do { } while (0)
#endif

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
__device__ __forceinline__ float ex2(float x) {
  float r;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(r) : "f"(x));
  return r;
}
__device__ __forceinline__ void softmax_bar() { asm volatile("bar.sync 1, 256;" ::: "memory"); }
// Barrier of the 256 softmax threads that also ANDs a flag, so that a wait given up by one
// warp ends the loop of all four and nobody is left waiting at a later barrier.
__device__ __forceinline__ bool softmax_bar_and(bool v) {
  uint32_t out;
  asm volatile(
      "{\n\t.reg .pred q, r;\n\t"
      "setp.ne.u32 q, %1, 0;\n\t"
      "bar.red.and.pred r, 1, 256, q;\n\t"
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
#ifdef FST_ATTN_TRACE
  CTA_TRACE(0, gtime());
  CTA_TRACE(4, clock64());
  CTA_TRACE(3, (long long)(seg1 - seg0));
#endif

  if (threadIdx.x == 0) {
    tc::mbar_init(&mi->q_full, 1);
    for (int c = 0; c < 9; ++c) {
      tc::mbar_init(&mi->kv_full[c], 1);
      tc::mbar_init(&mi->kv_empty[c], 1);
    }
    tc::mbar_init(&mi->s_full, 1);
    tc::mbar_init(&mi->p_full, SOFTMAX_THREADS);
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
  // everything above overlapped with the tail of the previous kernel; Q_eff and the appended
  // cache rows are its products
  pdl_launch();
  pdl_wait();
#ifdef FST_ATTN_TRACE
  CTA_TRACE(1, gtime());
#endif

  if (warp == 0 || warp >= 10) {
    // ---------------- TMA producers ----------------
    // Three producer warps (0, 10, 11), one lane each: a thread needs ~200 cycles per tensor
    // copy it issues, so the 18 copies of a tile are split three ways.  Producer r streams
    // chunks r, r+3, r+6: the SV MMAs free chunks 0-3 first and 4-8 last, and this way no
    // producer has more than two of the late chunks.
    if (lane == 0) {
      const int r = warp == 0 ? 0 : warp - 9;
      if (r == 0) {
        tc::tma_prefetch_desc(&tmQ);
        tc::tma_prefetch_desc(&tmKV);
      }
      // half of the CTAs start a little later, so that the SMs do not all refill their tile
      // (and compete for L2 bandwidth) at the same instant
      if (FST_STAGGER && (blockIdx.x & 1)) __nanosleep(FST_STAGGER);
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
          for (int c = r; c < NCH; c += 3) {
            if (g > 0) {
              ok = tc::mbar_wait(&mi->kv_empty[c], (g - 1) & 1, abort_flag, p.d_status, ST_TMA_TIMEOUT);
              if (!ok) break;
            }
            if (c == 0) TRACE(g, 0);
            if (t == 0) {
              // The QK MMAs of the previous segment have retired (they precede the SV MMAs that
              // freed this chunk), so Q_eff may be replaced.  Producer 0 arms the barrier; a copy
              // that completes before that only makes the pending byte count negative.
              if (c == 0) tc::mbar_expect_tx(&mi->q_full, L::Q_BYTES);
              tc::tma_load_3d(s_q + c * Q_CHUNK, &tmQ, &mi->q_full, c * 64, sg.tok * HEADS, 0);
            }
            tc::mbar_expect_tx(&mi->kv_full[c], KV_CHUNK);
            tc::tma_load_3d(s_kv + c * KV_CHUNK, &tmKV, &mi->kv_full[c], c * 64, row0, 0);
            tc::tma_load_3d(s_kv + c * KV_CHUNK + KV_CHUNK / 2, &tmKV, &mi->kv_full[c], c * 64, row1, 0);
            if (c == NCH - 1) TRACE(g, 1);
          }
          // Start the HBM reads of the NEXT tile of this segment now: its copies, issued as
          // chunks are freed, then hit L2.
          if (ok && FST_PREFETCH && base + TILE < sg.kv_end) {
            const int nrow0 = table[(base >> 6) + 2] * 64;
            const int nrow1 = base + TILE + 64 < sg.kv_end ? table[(base >> 6) + 3] * 64 : -1;
            for (int c = r; c < NCH; c += 3) {
              tc::tma_prefetch_3d(&tmKV, c * 64, nrow0, 0);
              if (nrow1 >= 0) tc::tma_prefetch_3d(&tmKV, c * 64, nrow1, 0);
            }
          }
        }
      }
    }
  } else if (warp == 1) {
    // ---------------- MMA issuer ----------------
    if (lane == 0) {
      constexpr uint32_t idesc_qk = tc::umma_idesc_bf16(TILE, HEADS, 0, 0);
      constexpr uint32_t idesc_sv = tc::umma_idesc_bf16(HEADS, 256, 1, 1);
      // descriptors differ only in their start-address field (16-byte units): the rest is constant
      const uint64_t k_major = tc::umma_desc_sw128(0, 16, 1024);
      const uint64_t vt_desc = tc::umma_desc_sw128(0, KV_CHUNK, 1024);
      const uint32_t q16 = (tc::smem_u32(s_q) & 0x3FFFFu) >> 4, kv16 = (tc::smem_u32(s_kv) & 0x3FFFFu) >> 4,
                     p16 = (tc::smem_u32(s_p) & 0x3FFFFu) >> 4;
      int g = 0, sidx = 0;
      bool ok = true;
      for (int si = seg0; si < seg1 && ok; ++si, ++sidx) {
        const AttnSeg sg = p.segs[si];
        const int n_tiles = (sg.kv_end - sg.kv_begin + TILE - 1) / TILE;
        ok = tc::mbar_wait(&mi->q_full, sidx & 1, abort_flag, p.d_status, ST_MMA_TIMEOUT);
        for (int t = 0; t < n_tiles && ok; ++t, ++g) {
          // S^T = K * Q^T, chunk by chunk as the tile lands
#pragma unroll
          for (int c = 0; c < NCH; ++c) {
            ok = tc::mbar_wait(&mi->kv_full[c], g & 1, abort_flag, p.d_status, ST_MMA_TIMEOUT);
            if (!ok) break;
            if (c == 0) TRACE(g, 2);
            if (c == NCH - 1) TRACE(g, 3);
            tc::tc_fence_after();
#pragma unroll
            for (int k = 0; k < 4; ++k) {
              const uint64_t da = k_major | (uint64_t)(kv16 + c * (KV_CHUNK / 16) + k * 2);
              const uint64_t db = k_major | (uint64_t)(q16 + c * (Q_CHUNK / 16) + k * 2);
              tc::umma_bf16(tmem + COL_S, da, db, idesc_qk, (c > 0 || k > 0) ? 1u : 0u);
            }
          }
          if (!ok) break;
          tc::umma_commit(&mi->s_full);
          TRACE(g, 4);
#ifdef FST_ATTN_TRACE
          tc::mbar_wait(&mi->s_full, g & 1, abort_flag, p.d_status, ST_MMA_TIMEOUT);
          TRACE(g, 14);  // QK MMAs retired
#endif
          // O^T += V^T * P^T once the softmax threads have written P^T
          ok = tc::mbar_wait(&mi->p_full, g & 1, abort_flag, p.d_status, ST_MMA_TIMEOUT);
          if (!ok) break;
          TRACE(g, 5);
          tc::tc_fence_after();
#pragma unroll
          for (int nh = 0; nh < 2; ++nh) {
#pragma unroll
            for (int k = 0; k < TILE / 16; ++k) {
              // A: P^T rows (tokens) 16k .. +15, all 64 heads.  B: the same tokens of latent
              // columns 256*nh .. +255 (chunks 4nh .. 4nh+3: LBO = chunk stride)
              const uint64_t da = k_major | (uint64_t)(p16 + k * 128);
              const uint64_t db = vt_desc | (uint64_t)(kv16 + 4 * nh * (KV_CHUNK / 16) + k * 128);
              tc::umma_bf16(tmem + COL_O + ((uint32_t)(nh * 16) << 16), da, db, idesc_sv, (t > 0 || k > 0) ? 1u : 0u);
            }
#pragma unroll
            for (int c = 0; c < 4; ++c) tc::umma_commit(&mi->kv_empty[4 * nh + c]);
          }
          if (NCH == 9) tc::umma_commit(&mi->kv_empty[8]);
          tc::umma_commit(&mi->o_done);
          TRACE(g, 6);
#ifdef FST_ATTN_TRACE
          tc::mbar_wait(&mi->o_done, g & 1, abort_flag, p.d_status, ST_MMA_TIMEOUT);
          TRACE(g, 7);  // SV MMAs retired
#endif
        }
      }
    }
  } else {
    // ---------------- softmax / epilogue ----------------
    // thread = one cached token of the tile (TMEM lane) and one half of the heads (32 columns)
    const int quad = warp & 3;            // TMEM lane quadrant this warp may touch
    const int half = (warp - 2) >> 2;     // heads 32*half .. 32*half+31
    const int tok_in_tile = quad * 32 + lane;
    const uint32_t lane_addr = tmem + ((uint32_t)(quad * 32) << 16);
    const int sm_tid = threadIdx.x - 64;  // 0..255
    const int h0 = half * 32;
    int g = 0;
    bool ok = true;
    for (int si = seg0; si < seg1 && ok; ++si) {
      const AttnSeg sg = p.segs[si];
      const int n_tiles = (sg.kv_end - sg.kv_begin + TILE - 1) / TILE;
      float l[32];
#pragma unroll
      for (int j = 0; j < 32; ++j) l[j] = 0.0f;
      if (sm_tid < HEADS) mi->m_used[sm_tid] = -INFINITY;
      softmax_bar();
      for (int t = 0; t < n_tiles && ok; ++t, ++g) {
        ok = tc::mbar_wait(&mi->s_full, g & 1, abort_flag, p.d_status, ST_SOFTMAX_TIMEOUT);
        if (sm_tid == 0) TRACE(g, 8);
        tc::tc_fence_after();
        const bool valid = sg.kv_begin + t * TILE + tok_in_tile < sg.kv_end;
        float s[32];
        tc::tmem_ld32(lane_addr + COL_S + h0, s);
        // pass 1: maxima over the warp's 32 tokens for its 32 heads
#pragma unroll
        for (int j = 0; j < 32; ++j) {
          s[j] = valid ? s[j] * p.scale_log2 : -INFINITY;
          const float r = redux_max(s[j]);
          if (lane == j) mi->wmax[quad][h0 + j] = r;
        }
        if (sm_tid == 0) TRACE(g, 9);
        ok = softmax_bar_and(ok);
        if (!ok) break;
        if (sm_tid == 0) TRACE(g, 10);
        // one thread per head decides whether the reference maximum moves
        if (sm_tid < HEADS) {
          const float tm = fmaxf(fmaxf(mi->wmax[0][sm_tid], mi->wmax[1][sm_tid]),
                                 fmaxf(mi->wmax[2][sm_tid], mi->wmax[3][sm_tid]));
          const float mo = mi->m_used[sm_tid];
          float a = 1.0f;
          if (tm > mo + RESCALE_THRESHOLD) {  // also the first tile (mo = -inf)
            a = ex2(mo - tm);
            mi->m_used[sm_tid] = tm;
            if (t > 0) mi->rescale = 1;
          }
          mi->alpha[sm_tid] = a;
        }
        softmax_bar();
        if (sm_tid == 0) TRACE(g, 11);
        const bool rescale = mi->rescale != 0;
        // pass 2: P = exp2(s - m), row sums, P^T into shared memory (MN-major, 128-byte swizzle)
        {
          uint32_t packed[16];
#pragma unroll
          for (int j4 = 0; j4 < 32; j4 += 4) {
            const float4 m4 = *reinterpret_cast<const float4*>(&mi->m_used[h0 + j4]);
            float pv[4];
            pv[0] = ex2(s[j4] - m4.x);      // masked tokens: ex2(-inf) = 0
            pv[1] = ex2(s[j4 + 1] - m4.y);
            pv[2] = ex2(s[j4 + 2] - m4.z);
            pv[3] = ex2(s[j4 + 3] - m4.w);
            if (rescale) {
              const float4 a4 = *reinterpret_cast<const float4*>(&mi->alpha[h0 + j4]);
              l[j4] *= a4.x;
              l[j4 + 1] *= a4.y;
              l[j4 + 2] *= a4.z;
              l[j4 + 3] *= a4.w;
            }
#pragma unroll
            for (int e = 0; e < 4; ++e) l[j4 + e] += pv[e];
            __nv_bfloat162 b0 = __floats2bfloat162_rn(pv[0], pv[1]);
            __nv_bfloat162 b1 = __floats2bfloat162_rn(pv[2], pv[3]);
            packed[j4 / 2] = *reinterpret_cast<uint32_t*>(&b0);
            packed[j4 / 2 + 1] = *reinterpret_cast<uint32_t*>(&b1);
          }
          unsigned char* prow = s_p + tok_in_tile * 128;
#pragma unroll
          for (int q4 = 0; q4 < 4; ++q4) {
            const int chunk = (half * 4 + q4) ^ (tok_in_tile & 7);
            *reinterpret_cast<uint4*>(prow + chunk * 16) =
                make_uint4(packed[q4 * 4], packed[q4 * 4 + 1], packed[q4 * 4 + 2], packed[q4 * 4 + 3]);
          }
        }
        // the reference maximum moved: rescale O.  A 32-lane TMEM load hands lanes 0-15 the
        // rows of the first accumulator and lanes 16-31 those of the second, so thread = one
        // head, one half of the latent columns; the two warps of a quadrant split the columns.
        // s_full of this tile implies that the SV MMAs of the previous tile have retired.
        if (rescale) {
          const float a = mi->alpha[quad * 16 + (lane & 15)];
#pragma unroll 1
          for (int c = 0; c < 4; ++c) {
            float o[32];
            const uint32_t addr = lane_addr + COL_O + half * 128 + c * 32;
            tc::tmem_ld32(addr, o);
#pragma unroll
            for (int j = 0; j < 32; ++j) o[j] *= a;
            tc::tmem_st32(addr, o);
          }
        }
        if (sm_tid == 0) TRACE(g, 12);
        tc::fence_proxy_async();
        tc::tc_fence_before();
        softmax_bar();  // every thread has read alpha / rescale before they are reset
        if (sm_tid == 0) TRACE(g, 13);
        if (sm_tid == 0) mi->rescale = 0;
        tc::mbar_arrive(&mi->p_full);
      }
      if (!ok) break;
      // ---- epilogue of the segment: un-normalised partial (max, sum, O) ----
      ok = tc::mbar_wait(&mi->o_done, (g - 1) & 1, abort_flag, p.d_status, ST_EPI_TIMEOUT);
      tc::tc_fence_after();
#pragma unroll
      for (int j = 0; j < 32; ++j) {
        const float v = warp_sum(l[j]);
        if (lane == j) mi->wmax[quad][h0 + j] = v;
      }
      ok = softmax_bar_and(ok);
      if (!ok) break;
      if (sm_tid < HEADS) {
        const float sum = mi->wmax[0][sm_tid] + mi->wmax[1][sm_tid] + mi->wmax[2][sm_tid] + mi->wmax[3][sm_tid];
        p.part_l[(long long)sg.part * HEADS + sm_tid] = sum;
        p.part_m[(long long)sg.part * HEADS + sm_tid] = mi->m_used[sm_tid] * 0.6931471805599453f;  // back to ln units
      }
      {
        const int head = quad * 16 + (lane & 15);
        float* po = p.part_o + ((long long)sg.part * HEADS + head) * D_V + (lane >> 4) * 256 + half * 128;
#pragma unroll 1
        for (int c = 0; c < 4; ++c) {
          float o[32];
          tc::tmem_ld32(lane_addr + COL_O + half * 128 + c * 32, o);
#pragma unroll
          for (int j = 0; j < 32; j += 4)
            *reinterpret_cast<float4*>(po + c * 32 + j) = make_float4(o[j], o[j + 1], o[j + 2], o[j + 3]);
        }
      }
      tc::tc_fence_before();
      softmax_bar();  // wmax / m_used are reused by the next segment
    }
  }

  tc::tc_fence_before();
  __syncthreads();
#ifdef FST_ATTN_TRACE
  CTA_TRACE(2, gtime());
  CTA_TRACE(5, clock64());
#endif
  if (*abort_flag) {
    for (int i = 0; i < 2000; ++i) __nanosleep(1000);  // let copies and MMAs in flight settle
  }
  if (warp == 1) {
    tc::tc_fence_after();
    tc::tmem_dealloc(tmem, TMEM_COLS);
  }
}

}  // namespace

#ifdef FST_ATTN_TRACE
extern "C" int fst_debug_read_attn_trace(long long* out) {
  return (int)cudaMemcpyFromSymbol(out, g_attn_trace, sizeof(long long) * 64 * 16);
}
extern "C" int fst_debug_read_attn_cta(long long* out) {
  return (int)cudaMemcpyFromSymbol(out, g_attn_cta, sizeof(long long) * 256 * 8);
}
#endif

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
  p.pool = a.pool;
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
    e = launch_pdl(k_attn_tc<9>, dim3(a.n_ctas), dim3(ATTN_THREADS), Smem<9>::TOTAL, st, 1, tmQ, tmKV, p);
    if (e != cudaSuccess) return e;
  } else {
    static bool set8 = false;
    if (!set8) {
      e = cudaFuncSetAttribute(k_attn_tc<8>, cudaFuncAttributeMaxDynamicSharedMemorySize, Smem<8>::TOTAL);
      if (e != cudaSuccess) return e;
      set8 = true;
    }
    e = launch_pdl(k_attn_tc<8>, dim3(a.n_ctas), dim3(ATTN_THREADS), Smem<8>::TOTAL, st, 1, tmQ, tmKV, p);
    if (e != cudaSuccess) return e;
  }
  return cudaGetLastError();
}

}  // namespace fst
