// Split-KV latent attention, second generation: Q_eff lives in TENSOR MEMORY.
//
// Same job as attn_tc.cu (QK, softmax, SV of process_mla, reference src/fst_engine.cpp:
// 3573-3683, over the paged bf16 cache) for 576-wide rows and 64 heads, but both products are
// in their natural orientation with the 64 heads as MMA M:
//   S[64 heads, 128 tok]  = Q[64, 576] * K^T   A = Q_eff: the 512 latent dims from TMEM, the 64 rope
//                                               dims from shared memory; B = one chunk of the tile,
//                                               K-major, N = 128 tokens
//   O[64 heads, 512]     += P[64, 128] * V     A = P (shared memory, K-major, written row by row by the
//                                               softmax threads); B = the same cache bytes read
//                                               MN-major, N = 256 latent columns at a time
// Moving Q_eff out of shared memory frees 64 KB: the cache tile (nine 16 KB chunks) now lives in
// a ring of TWELVE chunk slots, so the first chunks of the next tile land -- and their QK MMAs
// run -- while the softmax of the current tile is still working, and P has its own buffer, so
// the rope chunk is recycled right after QK.
//
// Tensor memory (512 columns).  A 64-row operand or accumulator occupies lanes 0-15 of each
// 32-lane quadrant (row r in lane 32*(r/16) + r%16).  An accumulator may also sit at lane offset
// 16; an A operand may not, and an MMA that takes A from tensor memory needs its accumulator on
// the same lanes as A.  Hence:
//   lanes  0-15: Q latent (bf16 pairs) in columns [0,256) | S buffer 0 in [256,384) | S buffer 1 in [384,512)
//   lanes 16-31: O[64, 512] in columns [0,512)  (its MMAs take A = P from shared memory)
// 32-lane accesses of the softmax threads are read-only wherever the other 16 lanes hold live
// data; O is rescaled through the 16-lane access shape.
//
// Softmax: a score row belongs to one head, so maxima and sums are per thread; the two warps of a
// quadrant split the 128 tokens of a tile and exchange one maximum per row through shared memory.
#include "kernels.cuh"
#include "tc_common.cuh"

namespace fst {

namespace {

constexpr int TILE = 128;
constexpr int HEADS = 64;
constexpr int D_V = 512;
constexpr int NCH = 9;                 // chunks of 64 dims per 576-wide row
constexpr int SLOTS = 12;              // ring of chunk slots
constexpr int KV_CHUNK = TILE * 128;   // 16 KB: [128 tok x 64 dims]
constexpr int QR_BYTES = HEADS * 128;  // Q rope chunk [64 heads x 64 dims]
constexpr int P_BYTES = HEADS * TILE * 2;
constexpr int NAT_THREADS = 384;
constexpr uint32_t TMEM_COLS = 512;
constexpr uint32_t COL_Q = 0, COL_S = 256, COL_O = 0;
constexpr uint32_t LANE16 = 16u << 16;
constexpr float RESCALE_THRESHOLD = 8.0f;

constexpr int OFF_RING = 0;
constexpr int OFF_QR = SLOTS * KV_CHUNK;
constexpr int OFF_P = OFF_QR + QR_BYTES;
constexpr int OFF_MISC = OFF_P + P_BYTES;
constexpr int MISC_BYTES = 2048;
constexpr int SMEM_TOTAL = OFF_MISC + MISC_BYTES + 1024;

struct NatParams {
  const bf16* q_eff;
  const int32_t* tables;
  const int32_t* tok_table;
  const AttnSeg* segs;
  const int32_t* cta_seg;
  float* part_m;
  float* part_l;
  float* part_o;
  int* d_status;
  int pool_rows;
  float scale_log2;
};

#ifdef FST_ATTN_TRACE
__device__ long long g_nat_trace[64 * 16];
#define NTRACE(tile, ev) do { if (blockIdx.x == 0 && (tile) < 64) g_nat_trace[(tile) * 16 + (ev)] = clock64(); } while (0)
#else
#define NTRACE(tile, ev) do { } while (0)
#endif

struct NatMisc {
  uint64_t full[SLOTS];
  uint64_t empty[SLOTS];
  uint64_t qr_full;      // Q rope chunk landed (TMA)
  uint64_t q_tmem;       // Q latent written to TMEM by the softmax threads
  uint64_t q_free;       // the QK MMAs of a segment have retired: Q may be replaced
  uint64_t s_full[2];
  uint64_t p_full;
  uint64_t o_done;
  uint32_t tmem_slot;
  int abort_flag;
  float pmax[2][HEADS];  // per token-half row maxima; row sums in the epilogue
};

__device__ __forceinline__ float ex2f(float x) {
  float r;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(r) : "f"(x));
  return r;
}
__device__ __forceinline__ void sm_bar() { asm volatile("bar.sync 1, 256;" ::: "memory"); }
__device__ __forceinline__ bool sm_bar_and(bool v) {
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
// 16 lanes x 64 columns: thread t < 16 gets lane (base + t), columns [c, c+32); thread t >= 16
// gets lane (base + t - 16), columns [c+32, c+64).
__device__ __forceinline__ void tmem_ld16x64(uint32_t taddr, float* v) {
  uint32_t r[32];
  asm volatile(
      "tcgen05.ld.sync.aligned.16x32bx2.x32.b32 "
      "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, "
      "%16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, [%32], 32;"
      : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]),
        "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]),
        "=r"(r[16]), "=r"(r[17]), "=r"(r[18]), "=r"(r[19]), "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]),
        "=r"(r[24]), "=r"(r[25]), "=r"(r[26]), "=r"(r[27]), "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
      : "r"(taddr)
      : "memory");
  asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
#pragma unroll
  for (int i = 0; i < 32; ++i) v[i] = __uint_as_float(r[i]);
}
__device__ __forceinline__ void tmem_st16x64(uint32_t taddr, const float* v) {
  asm volatile(
      "tcgen05.st.sync.aligned.16x32bx2.x32.b32 [%32], 32, "
      "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, "
      "%16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31};"
      ::"r"(__float_as_uint(v[0])), "r"(__float_as_uint(v[1])), "r"(__float_as_uint(v[2])), "r"(__float_as_uint(v[3])),
        "r"(__float_as_uint(v[4])), "r"(__float_as_uint(v[5])), "r"(__float_as_uint(v[6])), "r"(__float_as_uint(v[7])),
        "r"(__float_as_uint(v[8])), "r"(__float_as_uint(v[9])), "r"(__float_as_uint(v[10])), "r"(__float_as_uint(v[11])),
        "r"(__float_as_uint(v[12])), "r"(__float_as_uint(v[13])), "r"(__float_as_uint(v[14])), "r"(__float_as_uint(v[15])),
        "r"(__float_as_uint(v[16])), "r"(__float_as_uint(v[17])), "r"(__float_as_uint(v[18])), "r"(__float_as_uint(v[19])),
        "r"(__float_as_uint(v[20])), "r"(__float_as_uint(v[21])), "r"(__float_as_uint(v[22])), "r"(__float_as_uint(v[23])),
        "r"(__float_as_uint(v[24])), "r"(__float_as_uint(v[25])), "r"(__float_as_uint(v[26])), "r"(__float_as_uint(v[27])),
        "r"(__float_as_uint(v[28])), "r"(__float_as_uint(v[29])), "r"(__float_as_uint(v[30])), "r"(__float_as_uint(v[31])),
        "r"(taddr)
      : "memory");
  asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory");
}
// D[tmem] (+)= A[tmem] * B[smem]
__device__ __forceinline__ void umma_ts(uint32_t d_tmem, uint32_t a_tmem, uint64_t b_desc, uint32_t idesc, uint32_t acc) {
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], [%1], %2, %3, p;\n\t}"
      ::"r"(d_tmem), "r"(a_tmem), "l"(b_desc), "r"(idesc), "r"(acc)
      : "memory");
}


__global__ void __launch_bounds__(NAT_THREADS, 1)
k_attn_nat(const __grid_constant__ CUtensorMap tmQ, const __grid_constant__ CUtensorMap tmKV, NatParams p) {
  extern __shared__ __align__(1024) unsigned char smem_raw[];
  unsigned char* smem = reinterpret_cast<unsigned char*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  unsigned char* s_ring = smem + OFF_RING;
  unsigned char* s_qr = smem + OFF_QR;
  unsigned char* s_p = smem + OFF_P;
  NatMisc* mi = reinterpret_cast<NatMisc*>(smem + OFF_MISC);
  volatile int* abort_flag = &mi->abort_flag;

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int seg0 = p.cta_seg[blockIdx.x], seg1 = p.cta_seg[blockIdx.x + 1];

  if (threadIdx.x == 0) {
    for (int i = 0; i < SLOTS; ++i) {
      tc::mbar_init(&mi->full[i], 1);
      tc::mbar_init(&mi->empty[i], 1);
    }
    tc::mbar_init(&mi->qr_full, 1);
    tc::mbar_init(&mi->q_tmem, 256);
    tc::mbar_init(&mi->q_free, 1);
    tc::mbar_init(&mi->s_full[0], 1);
    tc::mbar_init(&mi->s_full[1], 1);
    tc::mbar_init(&mi->p_full, 256);
    tc::mbar_init(&mi->o_done, 1);
    mi->abort_flag = 0;
    tc::fence_barrier_init();
  }
  if (warp == 1) tc::tmem_alloc(&mi->tmem_slot, TMEM_COLS);
  tc::tc_fence_before();
  __syncthreads();
  tc::tc_fence_after();
  const uint32_t tmem = mi->tmem_slot;
  pdl_launch();
  pdl_wait();  // Q_eff and the appended cache rows come from earlier kernels

  if (warp == 0 || warp >= 10) {
    // ---------------- TMA producers: lane 0 of warps 0, 10, 11 ----------------
    // Producer r streams chunks r, r+3, r+6 of every tile into the ring, in ring order.
    if (lane == 0) {
      const int r = warp == 0 ? 0 : warp - 9;
      if (r == 0) {
        tc::tma_prefetch_desc(&tmQ);
        tc::tma_prefetch_desc(&tmKV);
      }
      int g = 0, sidx = 0;
      bool ok = true;
      for (int si = seg0; si < seg1 && ok; ++si, ++sidx) {
        const AttnSeg sg = p.segs[si];
        const int32_t* table = p.tables + p.tok_table[sg.tok];
        const int n_tiles = (sg.kv_end - sg.kv_begin + TILE - 1) / TILE;
        if (r == 0) {
          // the rope chunk of Q_eff; the previous segment's QK MMAs must have retired
          if (sidx > 0) ok = tc::mbar_wait(&mi->q_free, (sidx - 1) & 1, abort_flag, p.d_status, ST_TMA_TIMEOUT);
          if (!ok) break;
          tc::mbar_expect_tx(&mi->qr_full, QR_BYTES);
          tc::tma_load_3d(s_qr, &tmQ, &mi->qr_full, (NCH - 1) * 64, sg.tok * HEADS, 0);
        }
        for (int t = 0; t < n_tiles && ok; ++t, ++g) {
          const int base = sg.kv_begin + t * TILE;
          const int row0 = table[base >> 6] * 64;
          const int row1 = base + 64 < sg.kv_end ? table[(base >> 6) + 1] * 64 : p.pool_rows;
          for (int c = r; c < NCH; c += 3) {
            const int j = g * NCH + c, slot = j % SLOTS;
            if (j >= SLOTS) {
              ok = tc::mbar_wait(&mi->empty[slot], ((j / SLOTS) - 1) & 1, abort_flag, p.d_status, ST_TMA_TIMEOUT);
              if (!ok) break;
            }
            unsigned char* dst = s_ring + slot * KV_CHUNK;
            tc::mbar_expect_tx(&mi->full[slot], KV_CHUNK);
            tc::tma_load_3d(dst, &tmKV, &mi->full[slot], c * 64, row0, 0);
            tc::tma_load_3d(dst + KV_CHUNK / 2, &tmKV, &mi->full[slot], c * 64, row1, 0);
          }
          // bring the next tile of this segment into L2 meanwhile
          if (ok && base + TILE < sg.kv_end) {
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
      constexpr uint32_t idesc_qk = tc::umma_idesc_bf16(HEADS, TILE, 0, 0);
      const uint64_t k_major = tc::umma_desc_sw128(0, 16, 1024);
      const uint64_t v_desc = tc::umma_desc_sw128(0, KV_CHUNK, 1024);  // MN-major: 64-column groups one chunk apart
      const uint32_t ring16 = (tc::smem_u32(s_ring) & 0x3FFFFu) >> 4, qr16 = (tc::smem_u32(s_qr) & 0x3FFFFu) >> 4,
                     p16 = (tc::smem_u32(s_p) & 0x3FFFFu) >> 4;
      // QK MMAs of chunk c of ring tile gi into score buffer gi & 1
      auto qk_chunk = [&](int gi, int c) -> bool {
        const int j = gi * NCH + c, slot = j % SLOTS;
        if (!tc::mbar_wait(&mi->full[slot], (j / SLOTS) & 1, abort_flag, p.d_status, ST_MMA_TIMEOUT)) return false;
        tc::tc_fence_after();
        const uint32_t d = tmem + COL_S + (gi & 1) * TILE;  // same lanes as the TMEM-resident A
#pragma unroll
        for (int k = 0; k < 4; ++k) {
          const uint64_t db = k_major | (uint64_t)(ring16 + slot * (KV_CHUNK / 16) + k * 2);
          const uint32_t acc = (c > 0 || k > 0) ? 1u : 0u;
          if (c < NCH - 1)
            umma_ts(d, tmem + COL_Q + c * 32 + k * 8, db, idesc_qk, acc);  // 16 dims = 8 columns of bf16 pairs
          else
            tc::umma_bf16(d, k_major | (uint64_t)(qr16 + k * 2), db, idesc_qk, acc);
        }
        if (c == NCH - 1) tc::umma_commit(&mi->empty[slot]);  // the rope chunk is only a key
        return true;
      };
      int g = 0, sidx = 0;
      bool ok = true;
      for (int si = seg0; si < seg1 && ok; ++si, ++sidx) {
        const AttnSeg sg = p.segs[si];
        const int n_tiles = (sg.kv_end - sg.kv_begin + TILE - 1) / TILE;
        ok = tc::mbar_wait(&mi->qr_full, sidx & 1, abort_flag, p.d_status, ST_MMA_TIMEOUT) &&
             tc::mbar_wait(&mi->q_tmem, sidx & 1, abort_flag, p.d_status, ST_MMA_TIMEOUT);
        tc::tc_fence_after();
        int early = 0;  // chunks of tile g whose QK MMAs were issued during the previous tile
        for (int t = 0; t < n_tiles && ok; ++t, ++g) {
          NTRACE(g, 0);
          for (int c = early; c < NCH && ok; ++c) ok = qk_chunk(g, c);
          if (!ok) break;
          tc::umma_commit(&mi->s_full[g & 1]);
          NTRACE(g, 1);
          if (t == n_tiles - 1) tc::umma_commit(&mi->q_free);
          // while the softmax threads work on tile g: QK of the chunks of tile g+1 that fit in
          // the spare ring slots
          early = 0;
          if (t + 1 < n_tiles) {
            for (int c = 0; c < SLOTS - NCH && ok; ++c) ok = qk_chunk(g + 1, c);
            early = SLOTS - NCH;
          }
          if (!ok) break;
          NTRACE(g, 2);
          ok = tc::mbar_wait(&mi->p_full, g & 1, abort_flag, p.d_status, ST_MMA_TIMEOUT);
          if (!ok) break;
          NTRACE(g, 3);
          tc::tc_fence_after();
          // O += P * V: latent columns 256*nh .. +255 are chunks 4nh .. 4nh+3 of the tile; where
          // the ring wraps inside such a group the MMA is split at the wrap
#pragma unroll
          for (int nh = 0; nh < 2; ++nh) {
            const int s0 = (g * NCH + 4 * nh) % SLOTS;
            const int n1 = min(4, SLOTS - s0);
            const uint32_t d = tmem + LANE16 + COL_O + nh * 256;
            const uint32_t id1 = tc::umma_idesc_bf16(HEADS, n1 * 64, 0, 1), id2 = tc::umma_idesc_bf16(HEADS, (4 - n1) * 64, 0, 1);
#pragma unroll
            for (int k = 0; k < TILE / 16; ++k) {
              const uint64_t da = k_major | (uint64_t)(p16 + (k >> 2) * (P_BYTES / 32) + (k & 3) * 2);
              const uint32_t acc = (t > 0 || k > 0) ? 1u : 0u;
              tc::umma_bf16(d, da, v_desc | (uint64_t)(ring16 + s0 * (KV_CHUNK / 16) + k * 128), id1, acc);
              if (n1 < 4) tc::umma_bf16(d + n1 * 64, da, v_desc | (uint64_t)(ring16 + k * 128), id2, acc);
            }
            for (int c = 0; c < 4; ++c) tc::umma_commit(&mi->empty[(s0 + c) % SLOTS]);
          }
          tc::umma_commit(&mi->o_done);
          NTRACE(g, 4);
#ifdef FST_ATTN_TRACE
          tc::mbar_wait(&mi->o_done, g & 1, abort_flag, p.d_status, ST_MMA_TIMEOUT);
          NTRACE(g, 5);
#endif
        }
      }
    }
  } else {
    // ---------------- softmax / epilogue (warps 2-9) ----------------
    // A 32-lane TMEM load hands lanes 0-15 the score rows (row = head 16*quad + lane) and lanes
    // 16-31 the rows of O (lanes 16-31 idle through the softmax, lanes 0-15 through the
    // epilogue).  The two warps of a quadrant split a tile's 128 tokens (scores, P) and O's columns.
    const int quad = warp & 3;
    const int half = (warp - 2) >> 2;
    const int row = quad * 16 + (lane & 15);
    const bool active = lane < 16;
    const uint32_t lane_addr = tmem + ((uint32_t)(quad * 32) << 16);
    int g = 0, sidx = 0;
    bool ok = true;
    for (int si = seg0; si < seg1 && ok; ++si, ++sidx) {
      const AttnSeg sg = p.segs[si];
      const int n_tiles = (sg.kv_end - sg.kv_begin + TILE - 1) / TILE;
      // Q_eff latent dims -> TMEM (bf16 pairs, two per column): this warp writes dims
      // 256*half .. +255 of its 16 rows.  Lanes 16-31 of these columns belong to O, which holds
      // nothing between segments.
      {
        const uint4* src = reinterpret_cast<const uint4*>(p.q_eff + ((long long)sg.tok * HEADS + row) * (NCH * 64) + half * 256);
#pragma unroll 1
        for (int cc = 0; cc < 4; ++cc) {
          float w[32];
#pragma unroll
          for (int q4 = 0; q4 < 8; ++q4) {
            const uint4 v = src[cc * 8 + q4];
            w[q4 * 4] = __uint_as_float(v.x);
            w[q4 * 4 + 1] = __uint_as_float(v.y);
            w[q4 * 4 + 2] = __uint_as_float(v.z);
            w[q4 * 4 + 3] = __uint_as_float(v.w);
          }
          tc::tmem_st32(lane_addr + COL_Q + half * 128 + cc * 32, w);
        }
        tc::tc_fence_before();
        tc::mbar_arrive(&mi->q_tmem);
      }
      float m_used = -INFINITY, l = 0.0f;
      for (int t = 0; t < n_tiles && ok; ++t, ++g) {
        ok = tc::mbar_wait(&mi->s_full[g & 1], (g >> 1) & 1, abort_flag, p.d_status, ST_SOFTMAX_TIMEOUT);
        if (threadIdx.x == 64) NTRACE(g, 8);
        tc::tc_fence_after();
        const int tok0 = sg.kv_begin + t * TILE + half * 64;
        float sc[64];
        tc::tmem_ld32(lane_addr + COL_S + (g & 1) * TILE + half * 64, sc);
        tc::tmem_ld32(lane_addr + COL_S + (g & 1) * TILE + half * 64 + 32, sc + 32);
        float mx = -INFINITY;
#pragma unroll
        for (int j = 0; j < 64; ++j) {
          sc[j] = tok0 + j < sg.kv_end ? sc[j] * p.scale_log2 : -INFINITY;
          mx = fmaxf(mx, sc[j]);
        }
        if (active) mi->pmax[half][row] = mx;
        if (threadIdx.x == 64) NTRACE(g, 9);
        ok = sm_bar_and(ok);
        if (!ok) break;
        if (threadIdx.x == 64) NTRACE(g, 10);
        // the reference maximum moves only when the tile maximum exceeds it by more than 2^8
        const float tm = fmaxf(mi->pmax[0][row], mi->pmax[1][row]);
        float alpha = 1.0f;
        if (tm > m_used + RESCALE_THRESHOLD) {  // also the first tile (m_used = -inf)
          alpha = ex2f(m_used - tm);
          m_used = tm;
        }
        float sum = 0.0f;
        uint32_t packed[32];
#pragma unroll
        for (int j = 0; j < 64; j += 2) {
          const float p0 = ex2f(sc[j] - m_used), p1 = ex2f(sc[j + 1] - m_used);  // masked: ex2(-inf) = 0
          sum += p0 + p1;
          __nv_bfloat162 b = __floats2bfloat162_rn(p0, p1);
          packed[j / 2] = *reinterpret_cast<uint32_t*>(&b);
        }
        l = l * alpha + sum;
        if (active) {
          // P[row, 64*half .. +63]: one 128-byte row of K-major sub-chunk `half`, 128-byte swizzle
          unsigned char* prow = s_p + half * (P_BYTES / 2) + row * 128;
#pragma unroll
          for (int q4 = 0; q4 < 8; ++q4)
            *reinterpret_cast<uint4*>(prow + ((q4 ^ (row & 7)) * 16)) =
                make_uint4(packed[q4 * 4], packed[q4 * 4 + 1], packed[q4 * 4 + 2], packed[q4 * 4 + 3]);
        }
        // O rows are scaled by their own alpha, through the 16-lane access shape so that Q_eff
        // and the score buffers on the other 16 lanes are not touched: both half-warps address
        // O row lane%16, 32 columns each.  s_full of this tile implies that the SV MMAs of the
        // previous tile have retired.
        const float a_row = __shfl_sync(0xffffffffu, alpha, lane & 15);
        if (t > 0 && __any_sync(0xffffffffu, active && alpha != 1.0f)) {
#pragma unroll 1
          for (int cc = 0; cc < 4; ++cc) {
            float o[32];
            const uint32_t addr = lane_addr + LANE16 + COL_O + half * 256 + cc * 64;
            tmem_ld16x64(addr, o);
#pragma unroll
            for (int j = 0; j < 32; ++j) o[j] *= a_row;
            tmem_st16x64(addr, o);
          }
        }
        if (threadIdx.x == 64) NTRACE(g, 11);
        tc::fence_proxy_async();
        tc::tc_fence_before();
        tc::mbar_arrive(&mi->p_full);
      }
      if (!ok) break;
      // ---- epilogue of the segment: un-normalised partial (max, sum, O) ----
      ok = tc::mbar_wait(&mi->o_done, (g - 1) & 1, abort_flag, p.d_status, ST_EPI_TIMEOUT);
      tc::tc_fence_after();
      if (active) mi->pmax[half][row] = l;
      ok = sm_bar_and(ok);
      if (!ok) break;
      if (active && half == 0) {
        p.part_l[(long long)sg.part * HEADS + row] = mi->pmax[0][row] + mi->pmax[1][row];
        p.part_m[(long long)sg.part * HEADS + row] = m_used * 0.6931471805599453f;  // back to ln units
      }
      {
        // lanes 16-31 hold O row lane-16 of this quadrant; this warp writes columns 256*half .. +255
        float* po = p.part_o + ((long long)sg.part * HEADS + row) * D_V + half * 256;
#pragma unroll 1
        for (int cc = 0; cc < 8; ++cc) {
          float o[32];
          tc::tmem_ld32(lane_addr + COL_O + half * 256 + cc * 32, o);
          if (!active) {
#pragma unroll
            for (int j = 0; j < 32; j += 4)
              *reinterpret_cast<float4*>(po + cc * 32 + j) = make_float4(o[j], o[j + 1], o[j + 2], o[j + 3]);
          }
        }
      }
      tc::tc_fence_before();
      sm_bar();  // pmax, the score buffers and O are reused by the next segment
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

#ifdef FST_ATTN_TRACE
extern "C" int fst_debug_read_nat_trace(long long* out) {
  return (int)cudaMemcpyFromSymbol(out, g_nat_trace, sizeof(long long) * 64 * 16);
}
#endif

bool attn_nat_supported(const AttnArgs& a) {
  return a.H == HEADS && a.d_v == D_V && a.page_tokens == 64 && a.row == a.d_qk && a.d_qk == NCH * 64 &&
         a.pool_rows < (1ll << 31) && (reinterpret_cast<uintptr_t>(a.pool) & 15) == 0 &&
         (reinterpret_cast<uintptr_t>(a.q_eff) & 15) == 0;
}

cudaError_t launch_attn_nat(const AttnArgs& a, cudaStream_t st) {
  static_assert(sizeof(NatMisc) <= MISC_BYTES, "misc region too small");
  static_assert(SMEM_TOTAL <= 227 * 1024, "shared memory budget");
  if (a.n_segs <= 0) return cudaSuccess;
  CUtensorMap tmQ, tmKV;
  const char* err = nullptr;
  if (!tc::cached_tmap(&tmQ, a.q_eff, (uint64_t)a.d_qk, (uint64_t)a.q_rows, 1, (uint64_t)a.d_qk * 2,
                       (uint64_t)a.d_qk * 2 * (uint64_t)a.q_rows, 64, 64, 1, &err) ||
      !tc::cached_tmap(&tmKV, a.pool, (uint64_t)a.row, (uint64_t)a.pool_rows, 1, (uint64_t)a.row * 2,
                       (uint64_t)a.row * 2 * (uint64_t)a.pool_rows, 64, 64, 1, &err))
    return cudaErrorInvalidValue;
  NatParams p;
  p.q_eff = a.q_eff; p.tables = a.tables; p.tok_table = a.tok_table; p.segs = a.segs; p.cta_seg = a.cta_seg;
  p.part_m = a.part_m; p.part_l = a.part_l; p.part_o = a.part_o; p.d_status = a.d_status;
  p.pool_rows = (int)a.pool_rows;
  p.scale_log2 = a.scale * 1.4426950408889634f;
  static bool attr_set = false;
  if (!attr_set) {
    cudaError_t e = cudaFuncSetAttribute(k_attn_nat, cudaFuncAttributeMaxDynamicSharedMemorySize, SMEM_TOTAL);
    if (e != cudaSuccess) return e;
    attr_set = true;
  }
  return launch_pdl(k_attn_nat, dim3(a.n_ctas), dim3(NAT_THREADS), SMEM_TOTAL, st, 1, tmQ, tmKV, p);
}

}  // namespace fst
