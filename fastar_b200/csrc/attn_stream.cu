// Split-KV latent attention as a STREAM of 64-token tiles; Q_eff lives in tensor memory.
//
// QK, softmax and SV of process_mla (reference src/fst_engine.cpp:3573-3683) over the paged bf16
// cache, 64 heads, 512- or 576-wide rows.  Both products are in
// their natural orientation with the 64 heads as MMA M:
//   S[64 heads, 64 tok]   = Q[64, d_qk] * K^T   A = Q_eff from TENSOR MEMORY; B = one 8 KB chunk
//                                               [64 tok x 64 dims] of the page, K-major
//   O[64 heads, 512]     += P[64, 64] * V       A = P (shared memory, K-major, written by the softmax
//                                               threads); B = the same chunks read MN-major, N = 256
//                                               latent columns (four chunks) at a time
//
// Why 64-token tiles.  The kernel is bound by how many cache bytes an SM can keep in flight: a
// chunk occupies shared memory from the moment its copy is issued until the SV MMAs of its tile
// have retired.  With 128-token tiles one tile (144 KB) fills the SM, so copies, MMAs and softmax
// take turns.  A page-sized tile is 72 KB; with Q_eff out of shared memory the ring holds three
// tiles, so the copies of the next tiles are in flight while this one is computed.
//
// MMA issue.  One thread issues a tcgen05.mma about every 50-80 cycles whatever its size, and a
// 64-token tile needs 36 QK MMAs (K = 16 each) and 8 SV MMAs: there are two QK issuers (each
// accumulates half of the chunks of every tile into a score buffer of its own) and one SV issuer.
// They touch different accumulators and are ordered against each other only through the mbarriers
// of the softmax hand-off.
//
// Tensor memory (512 columns).  A 64-row operand or accumulator occupies lanes 0-15 of each
// 32-lane quadrant (row r in lane 32*(r/16) + r%16).  An accumulator may also sit at lane offset
// 16; an A operand may not, and an MMA that takes A from tensor memory needs its accumulator on
// the same lanes as A.  Hence:
//   lanes  0-15: Q_eff (bf16 pairs) in columns [0, d_qk/2) | three score buffers of 64 columns behind it
//   lanes 16-31: O[64, 512] in columns [0,512)  (its MMAs take A = P from shared memory)
// The softmax threads touch lanes 0-15 only through the 16-lane access shape (O is rescaled the
// same way at lane offset 16); 32-lane loads are used where the other 16 lanes are only read.
#include "kernels.cuh"
#include "tc_common.cuh"

namespace fst {

namespace {

constexpr int TILE = 64;               // tokens per tile = one cache page
constexpr int HEADS = 64;
constexpr int D_V = 512;
constexpr int CHUNK = TILE * 128;      // 8 KB: [64 tok x 64 dims]
constexpr int P_BYTES = HEADS * TILE * 2;  // 8 KB
constexpr int ST_THREADS = 448;  // warps: 0, 10, 11 copy; 1, 13 issue QK; 12 issues SV; 2-9 softmax
constexpr uint32_t TMEM_COLS = 512;
constexpr uint32_t COL_Q = 0, COL_S = 288, COL_O = 0;
constexpr uint32_t LANE16 = 16u << 16;
constexpr float RESCALE_THRESHOLD = 8.0f;

// Shared memory: a ring of three tile frames (NCH chunk slots each); with eight chunks per tile
// three P buffers behind it (with nine, P lives in the frame's ninth chunk, see below); the
// staging area of the epilogue; barriers and small arrays.  227 KB either way.
//
// Where P lives.  The probabilities of a tile (64 heads x 64 tokens bf16, 8 KB) are the A operand
// of its SV MMAs.  Every tile has a P buffer of its own, with the life of its ring frame: for
// 576-wide rows it is the frame's ninth chunk -- the 64 rope dims, which only the QK MMAs read
// and which are dead once the tile's scores are complete; for 512-wide rows (eight chunks per
// tile, 24 KB of shared memory to spare) three buffers behind the ring.  So the softmax of the
// next tile stores its result without waiting for the SV MMAs of this one (with one shared P
// buffer it had to); it waits for them only in the rare case that it rescales O.  Worth 1.3 us
// of 85 on the batched-decode workload: the kernel is not bound by that dependency.
constexpr int MISC_BYTES = 2048;
constexpr int STAGE_BYTES = 8192;
__host__ __device__ constexpr int off_pbuf(int nch) { return 3 * nch * CHUNK; }
__host__ __device__ constexpr int off_stage(int nch) { return 3 * nch * CHUNK + (nch == 9 ? 0 : 3 * P_BYTES); }
__host__ __device__ constexpr int off_misc(int nch) { return off_stage(nch) + STAGE_BYTES; }
__host__ __device__ constexpr int smem_total(int nch) { return off_misc(nch) + MISC_BYTES + 1024; }
// byte offset (from the ring base) of the P buffer of the tile in ring slot g
template <int NCH>
__device__ __forceinline__ int p_slot_off(int g) {
  return NCH == 9 ? ((g % 3) * NCH + 8) * CHUNK : off_pbuf(NCH) + (g % 3) * P_BYTES;
}

struct StreamParams {
  const bf16* q_eff;
  const int32_t* tables;
  const AttnSeg* segs;
  const int32_t* cta_seg;
  const bf16* pool;
  float* part_m;
  float* part_l;
  float* part_o;
  int* d_status;
  int d_qk;
  float scale_log2;
  // direct != 0: a token whose whole context is one segment (one partial) is finished here --
  // normalised, rounded, (V4) inverse-rotated and written to o_lat -- and leaves no partial; the
  // merge kernel then skips it (see finish_token below)
  int direct;
  const int32_t* tok_part;  // [T + 1] partial slots of every token
  bf16* o_lat;              // [T * 64, 512]
  const float* sinks;       // [64] or null
  const float* lut;         // [T, rope] (cos, sin): inverse RoPE of the output tail of heads 0 .. inv_rope-1
  int rope, inv_rope;
  int tiles_shared;  // other blocks read the same tiles at about the same time: normal L2 priority
};


struct StreamMisc {
  uint64_t full_t[4][3]; // chunks 3i .. 3i+2 of tile g have landed: barrier [g & 3][i]
  uint64_t o_done[4];    // the SV MMAs of tile g have retired (its ring slots are free): barrier g & 3
  uint64_t q_ready;      // Q_eff of a segment written to tensor memory by the softmax threads
  uint64_t s_full[3];    // both score partials of tile n are complete: barrier n & 1 (two commits); WHOLE: the
                         // scores of tile n, barrier n % 3 -- one per buffer, as the QK MMAs may run three tiles ahead
  uint64_t s_free[3];    // the softmax threads have read the partial in this score buffer
  uint64_t p_full[3];    // the probabilities of tile n are written: barrier n % 3
  uint32_t tmem_slot;
  int abort_flag;
  float pmax[2][2][HEADS];  // [tile parity][token half][head]: row maxima of the two warps of a quadrant
  float lsum[2][HEADS];     // [token half][head]: row sums, in the epilogue
};

__device__ __forceinline__ float ex2f(float x) {
  float r;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(r) : "f"(x));
  return r;
}
// Barrier of the two warps of one quadrant (64 threads) that also ANDs a predicate.
__device__ __forceinline__ bool quad_bar_and(int quad, bool v) {
  uint32_t out;
  asm volatile(
      "{\n\t.reg .pred q, r;\n\t"
      "setp.ne.u32 q, %2, 0;\n\t"
      "bar.red.and.pred r, %1, 64, q;\n\t"
      "selp.u32 %0, 1, 0, r;\n\t}"
      : "=r"(out)
      : "r"(2 + quad), "r"((uint32_t)v)
      : "memory");
  return out != 0;
}

// 16-lane tensor-memory access (shape 16x32bx2): threads 0-15 of the warp address lanes
// base .. base+15, columns [c, c+N/2); threads 16-31 address the SAME lanes, columns
// [c+N/2, c+N), where N is 64 (x32) or 32 (x16).  Lanes base+16 .. base+31 are not touched.
__device__ __forceinline__ void tmem_ld16x64(uint32_t taddr, float* v) {
  uint32_t r[32];
  asm volatile("tcgen05.ld.sync.aligned.16x32bx2.x32.b32 {%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, %16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, [%32], 32;"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]), "=r"(r[16]), "=r"(r[17]), "=r"(r[18]), "=r"(r[19]), "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]), "=r"(r[24]), "=r"(r[25]), "=r"(r[26]), "=r"(r[27]), "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
               : "r"(taddr)
               : "memory");
  asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
#pragma unroll
  for (int i = 0; i < 32; ++i) v[i] = __uint_as_float(r[i]);
}
__device__ __forceinline__ void tmem_st16x64(uint32_t taddr, const float* v) {
  asm volatile("tcgen05.st.sync.aligned.16x32bx2.x32.b32 [%32], 32, {%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, %16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31};"
               ::"r"(__float_as_uint(v[0])), "r"(__float_as_uint(v[1])), "r"(__float_as_uint(v[2])), "r"(__float_as_uint(v[3])), "r"(__float_as_uint(v[4])), "r"(__float_as_uint(v[5])), "r"(__float_as_uint(v[6])), "r"(__float_as_uint(v[7])), "r"(__float_as_uint(v[8])), "r"(__float_as_uint(v[9])), "r"(__float_as_uint(v[10])), "r"(__float_as_uint(v[11])), "r"(__float_as_uint(v[12])), "r"(__float_as_uint(v[13])), "r"(__float_as_uint(v[14])), "r"(__float_as_uint(v[15])), "r"(__float_as_uint(v[16])), "r"(__float_as_uint(v[17])), "r"(__float_as_uint(v[18])), "r"(__float_as_uint(v[19])), "r"(__float_as_uint(v[20])), "r"(__float_as_uint(v[21])), "r"(__float_as_uint(v[22])), "r"(__float_as_uint(v[23])), "r"(__float_as_uint(v[24])), "r"(__float_as_uint(v[25])), "r"(__float_as_uint(v[26])), "r"(__float_as_uint(v[27])), "r"(__float_as_uint(v[28])), "r"(__float_as_uint(v[29])), "r"(__float_as_uint(v[30])), "r"(__float_as_uint(v[31])), "r"(taddr)
               : "memory");
}
__device__ __forceinline__ void tmem_ld16x32(uint32_t taddr, float* v) {
  uint32_t r[16];
  asm volatile("tcgen05.ld.sync.aligned.16x32bx2.x16.b32 {%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15}, [%16], 16;"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15])
               : "r"(taddr)
               : "memory");
  asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
#pragma unroll
  for (int i = 0; i < 16; ++i) v[i] = __uint_as_float(r[i]);
}
__device__ __forceinline__ void tmem_st16x32(uint32_t taddr, const float* v) {
  asm volatile("tcgen05.st.sync.aligned.16x32bx2.x16.b32 [%16], 16, {%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15};"
               ::"r"(__float_as_uint(v[0])), "r"(__float_as_uint(v[1])), "r"(__float_as_uint(v[2])), "r"(__float_as_uint(v[3])), "r"(__float_as_uint(v[4])), "r"(__float_as_uint(v[5])), "r"(__float_as_uint(v[6])), "r"(__float_as_uint(v[7])), "r"(__float_as_uint(v[8])), "r"(__float_as_uint(v[9])), "r"(__float_as_uint(v[10])), "r"(__float_as_uint(v[11])), "r"(__float_as_uint(v[12])), "r"(__float_as_uint(v[13])), "r"(__float_as_uint(v[14])), "r"(__float_as_uint(v[15])), "r"(taddr)
               : "memory");
}
__device__ __forceinline__ void tmem_wait_st() { asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory"); }
// D[tmem] (+)= A[tmem] * B[smem]
__device__ __forceinline__ void umma_ts(uint32_t d_tmem, uint32_t a_tmem, uint64_t b_desc, uint32_t idesc, uint32_t acc) {
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], [%1], %2, %3, p;\n\t}"
      ::"r"(d_tmem), "r"(a_tmem), "l"(b_desc), "r"(idesc), "r"(acc)
      : "memory");
}

// Walks the tiles of a CTA's segment list in order: every role keeps one of these per stream
// position it tracks, so that all roles agree on (segment, tile in segment, running tile index).
// The ring carries SLOTS: every segment puts its Q_eff block (64 heads x d_qk, the geometry of a
// page) into one slot, followed by one slot per tile.
struct TileCursor {
  int si, seg_end;   // current segment, one past the CTA's last
  int t, n_tiles;    // tile within the segment, tiles of the segment
  int g;             // running slot index over the whole list (ring frame g % 3)
  int gq;            // slot of the current segment's Q_eff block
  int n;             // running tile index (slots that are tiles)
  int sidx;          // running segment index
  AttnSeg sg;
  __device__ __forceinline__ void load(const AttnSeg* segs) {
    if (si < seg_end) {
      sg = segs[si];
      // kv_begin is page aligned except at the edge of a sliding window
      n_tiles = (sg.kv_end - (sg.kv_begin & ~(TILE - 1)) + TILE - 1) / TILE;
      gq = g++;
    }
  }
  __device__ __forceinline__ void init(const AttnSeg* segs, int seg0, int seg1) {
    si = seg0; seg_end = seg1; t = 0; g = 0; gq = 0; n = 0; sidx = 0; n_tiles = 0;
    load(segs);
  }
  __device__ __forceinline__ bool done() const { return si >= seg_end; }
  __device__ __forceinline__ void next(const AttnSeg* segs) {
    ++g; ++n;
    if (++t == n_tiles) {
      t = 0; ++si; ++sidx;
      load(segs);
    }
  }
};

// A token whose whole context was one segment needs no merge: its output row goes from tensor
// memory straight to o_lat, with the arithmetic the merge kernels apply to a single part --
// out = e^{m - M} O / (e^{m - M} l [+ e^{sink - M}] + 1e-12) with M = max(m, sink), rounded to bf16,
// then (V4) the inverse RoPE of the output tail (reference src/fst_engine.cpp:3623, 3636, 3646,
// 3716).  Run by the eight softmax warps; a thread owns 32 columns of one head (the 16-lane
// tensor-memory access shape).
__device__ __forceinline__ void finish_token(const StreamParams& p, int tok, int row, int half, int sub,
                                             uint32_t lane_addr, float m_ln, float l_row) {
  const bool sk = p.sinks != nullptr;
  const float M = sk ? fmaxf(p.sinks[row], m_ln) : m_ln;
  const float w = m_ln == -INFINITY ? 0.0f : expf(m_ln - M);
  float den = sk ? expf(p.sinks[row] - M) : 0.0f;
  if (m_ln != -INFINITY) den += w * l_row;
  const float inv = den > 0.0f ? 1.0f / (den + 1e-12f) : 0.0f;
  const float* lut = p.lut + (long long)tok * p.rope;
  bf16* o_row = p.o_lat + ((long long)tok * HEADS + row) * D_V;
#pragma unroll 1
  for (int cc = 0; cc < 4; ++cc) {
    const int col0 = half * 256 + cc * 64 + sub * 32;
    float o[32];
    tmem_ld16x64(lane_addr + LANE16 + COL_O + half * 256 + cc * 64, o);
#pragma unroll
    for (int j = 0; j < 32; ++j) o[j] = rbf(fmaf(w, o[j], 0.0f) * inv);
    if (row < p.inv_rope && col0 + 32 > D_V - p.rope) {
      // inverse RoPE of the rounded output tail: pairs (2i, 2i+1) sit in one thread
#pragma unroll
      for (int j = 0; j < 32; j += 2) {
        const int pr = col0 + j - (D_V - p.rope);
        if (pr >= 0) {
          const float c = lut[pr], sn = -lut[pr + 1], x0 = o[j], x1 = o[j + 1];
          o[j] = x0 * c - x1 * sn;
          o[j + 1] = x0 * sn + x1 * c;
        }
      }
    }
#pragma unroll
    for (int u = 0; u < 4; ++u) {
      uint32_t pk[4];
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        __nv_bfloat162 b2 = __floats2bfloat162_rn(o[8 * u + 2 * e], o[8 * u + 2 * e + 1]);
        pk[e] = *reinterpret_cast<uint32_t*>(&b2);
      }
      *reinterpret_cast<uint4*>(o_row + col0 + 8 * u) = make_uint4(pk[0], pk[1], pk[2], pk[3]);
    }
  }
}

// The QK MMAs of chunks [C0, C1) of tile g: S_partial = Q[:, chunks] * K[:, chunks]^T.  Chunks land
// in groups of three, each group with a barrier.
template <int C0, int C1>
__device__ __forceinline__ bool qk_chunks(StreamMisc* mi, int g, uint32_t d, uint32_t tmem, uint32_t frame16,
                                          volatile int* abort_flag, int* d_status) {
  constexpr uint32_t idesc_qk = tc::umma_idesc_bf16(HEADS, TILE, 0, 0);
  const uint64_t k_major = tc::umma_desc_sw128(0, 16, 1024);
#pragma unroll
  for (int c = C0; c < C1; ++c) {
    if (c == C0 || c % 3 == 0) {
      if (!tc::mbar_wait(&mi->full_t[g & 3][c / 3], (g >> 2) & 1, abort_flag, d_status, ST_MMA_TIMEOUT)) return false;
      tc::tc_fence_after();
    }
    const uint64_t db = k_major | (uint64_t)(frame16 + c * (CHUNK / 16));
#pragma unroll
    for (int k = 0; k < 4; ++k)
      umma_ts(d, tmem + COL_Q + c * 32 + k * 8, db + k * 2, idesc_qk, (c > C0 || k > 0) ? 1u : 0u);
  }
  return true;
}

// 14 warps are allocated as 16 (granularity four): 128 registers per thread
// DIRECT: tokens with a single partial are finished here (finish_token); the variant without it is
// the one batched decode runs, where every token is split (the mere presence of that code in the
// kernel costs 2-3 us of 85 there, measured).
// WHOLE: each QK issuer takes whole tiles (alternating) into one score buffer per tile, instead of
// half of every tile's chunks into a buffer of its own.  A tile's scores then take longer to
// complete, but three buffers hold three tiles, so the QK MMAs run ahead of the softmax instead of
// waiting for it to free a buffer -- the better trade when tiles come from L2 (blocks of query
// tokens: the kernel is bound by its own pipeline there; attention of the 32 x 16 x 16384 verify block
// 1.69 -> 1.55 ms), the worse one when the life of a frame bounds the kernel (decode: 86 -> 88 us).
template <int NCH, bool DIRECT, bool WHOLE>
__global__ void __launch_bounds__(ST_THREADS, 1)
k_attn_stream(const __grid_constant__ CUtensorMap tmKV, const __grid_constant__ CUtensorMap tmQ, StreamParams p) {
  extern __shared__ __align__(1024) unsigned char smem_raw[];
  unsigned char* smem = reinterpret_cast<unsigned char*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  unsigned char* s_ring = smem;
  unsigned char* s_stage = smem + off_stage(NCH);
  StreamMisc* mi = reinterpret_cast<StreamMisc*>(smem + off_misc(NCH));
  volatile int* abort_flag = &mi->abort_flag;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int seg0 = p.cta_seg[blockIdx.x], seg1 = p.cta_seg[blockIdx.x + 1];

  if (threadIdx.x == 0) {
    for (int i = 0; i < 4; ++i) {
      for (int j = 0; j < 3; ++j) tc::mbar_init(&mi->full_t[i][j], j < 2 ? 3 : NCH - 6);
      tc::mbar_init(&mi->o_done[i], 1);
    }
    tc::mbar_init(&mi->q_ready, 256);
    for (int i = 0; i < 3; ++i) tc::mbar_init(&mi->s_full[i], WHOLE ? 1 : 2);
    for (int i = 0; i < 3; ++i) tc::mbar_init(&mi->s_free[i], 256);
    for (int i = 0; i < 3; ++i) tc::mbar_init(&mi->p_full[i], 256);
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

  if (warp == 0 || warp == 10 || warp == 11) {
    // ---------------- TMA producers: lane 0 of warps 0, 10, 11 ----------------
    // Tile g goes to ring frame g % 3, which is free once the SV MMAs of tile g-3 have retired;
    // chunk c of the tile is copied by producer (g * NCH + c) % 3.  The chunks of a tile land in three groups (one
    // chunk of each producer per group), each with its own barrier, so that the QK MMAs of the
    // first group run while the rest of the tile is still on its way.
    if (lane == 0) {
      const int r = warp == 0 ? 0 : warp - 9;
      if (r == 0) {
        tc::tma_prefetch_desc(&tmKV);
        tc::tma_prefetch_desc(&tmQ);
      }
      TileCursor cur;
      cur.init(p.segs, seg0, seg1);
      bool ok = true;
      // cache tiles are read once and are more than L2 holds: they leave L2 first, so that the
      // partials written here are still there when the merge reads them -- unless the schedule
      // has the lanes of a group read the same tiles side by side (blocks of query tokens)
      const uint64_t stream_policy = p.tiles_shared ? tc::l2_policy_evict_normal() : tc::l2_policy_evict_first();
      // the chunks of slot g that this producer copies, from rows row0 .. row0+63 of `map`
      auto fill = [&](int g, const CUtensorMap* map, int row0) -> bool {
        const int c0 = (r + 3 - (g * NCH) % 3) % 3;
        if (g >= 3 && !tc::mbar_wait(&mi->o_done[(g - 3) & 3], ((g - 3) >> 2) & 1, abort_flag, p.d_status, ST_TMA_TIMEOUT))
          return false;
        for (int c = c0; c < NCH; c += 3) {
          const int slot = (g % 3) * NCH + c;
          tc::mbar_expect_tx(&mi->full_t[g & 3][c / 3], CHUNK);
          tc::tma_load_3d_hint(s_ring + slot * CHUNK, map, &mi->full_t[g & 3][c / 3], c * 64, row0, 0, stream_policy);
        }
        return true;
      };
      while (!cur.done() && ok) {
        // a segment opens with the Q_eff block of its token (64 rows of q_eff)
        if (cur.t == 0) {
          ok = fill(cur.gq, &tmQ, cur.sg.tok * HEADS);
          if (!ok) break;
        }
        const int32_t* table = p.tables + cur.sg.table;
        const int row0 = table[(cur.sg.kv_begin >> 6) + cur.t] * TILE;
        ok = fill(cur.g, &tmKV, row0);
        cur.next(p.segs);
      }
    }
  } else if (warp == 1 || warp == 13) {
    // ---------------- QK issuers ----------------
    // A thread issues a tcgen05.mma about every 50-80 cycles, whatever its size, and needs a few
    // hundred cycles per barrier it waits on, so the 36 QK MMAs of a tile are split: warp 1
    // accumulates chunks 0-4 and warp 13 chunks 5-8 into score buffers of their own (the
    // softmax threads add the two).  Partial k = 2g + part lives in buffer k % 3.
    if (lane == 0) {
      const int part = warp == 1 ? 0 : 1;
      const uint32_t ring16 = (tc::smem_u32(s_ring) & 0x3FFFFu) >> 4;
      TileCursor cur;
      cur.init(p.segs, seg0, seg1);
      bool ok = true;
      while (!cur.done() && ok) {
        const int g = cur.g, n = cur.n;
        // both issuers wait for Q_eff of every segment; all softmax threads have read the block's
        // frame by then, which is what the producers wait for before they reuse it
        if (cur.t == 0) {
          ok = tc::mbar_wait(&mi->q_ready, cur.sidx & 1, abort_flag, p.d_status, ST_MMA_TIMEOUT);
          if (ok && part == 0) tc::mbar_arrive(&mi->o_done[cur.gq & 3]);
        }
        if (WHOLE && (n & 1) != part) {  // the other issuer's tile
          cur.next(p.segs);
          continue;
        }
        const int k = WHOLE ? n : 2 * n + part, buf = k % 3, use = k / 3;
        // the softmax threads have read the previous partial in this buffer
        if (ok && use >= 1) ok = tc::mbar_wait(&mi->s_free[buf], (use - 1) & 1, abort_flag, p.d_status, ST_MMA_TIMEOUT);
        if (!ok) break;
        const uint32_t d = tmem + COL_S + buf * TILE;  // same lanes as the TMEM-resident A
        const uint32_t frame16 = ring16 + (g % 3) * NCH * (CHUNK / 16);
        if (WHOLE) ok = qk_chunks<0, NCH>(mi, g, d, tmem, frame16, abort_flag, p.d_status);
        else if (part == 0) ok = qk_chunks<0, 5>(mi, g, d, tmem, frame16, abort_flag, p.d_status);
        else ok = qk_chunks<5, NCH>(mi, g, d, tmem, frame16, abort_flag, p.d_status);
        if (!ok) break;
        tc::umma_commit(&mi->s_full[WHOLE ? n % 3 : n & 1]);
        cur.next(p.segs);
      }
    }
  } else if (warp == 12) {
    // ---------------- SV issuer ----------------
    if (lane == 0) {
      const uint64_t k_major = tc::umma_desc_sw128(0, 16, 1024);
      const uint64_t v_desc = tc::umma_desc_sw128(0, CHUNK, 1024);  // MN-major: 64-column groups one slot apart
      const uint32_t ring16 = (tc::smem_u32(s_ring) & 0x3FFFFu) >> 4;
      constexpr uint32_t id256 = tc::umma_idesc_bf16(HEADS, 256, 0, 1);
      TileCursor cur;
      cur.init(p.segs, seg0, seg1);
      bool ok = true;
      while (!cur.done() && ok) {
        const int g = cur.g;
        ok = tc::mbar_wait(&mi->p_full[cur.n % 3], (cur.n / 3) & 1, abort_flag, p.d_status, ST_MMA_TIMEOUT);
        if (!ok) break;
        tc::tc_fence_after();
        const uint64_t da = k_major | (uint64_t)(ring16 + (p_slot_off<NCH>(g) >> 4));
        const uint32_t acc0 = cur.t > 0 ? 1u : 0u;
#pragma unroll
        for (int nh = 0; nh < 2; ++nh) {
          // latent columns 256*nh .. +255 are chunks 4nh .. 4nh+3 of the tile's frame
          const uint32_t d = tmem + LANE16 + COL_O + nh * 256;
          const uint64_t db = v_desc | (uint64_t)(ring16 + ((g % 3) * NCH + 4 * nh) * (CHUNK / 16));
#pragma unroll
          for (int k = 0; k < TILE / 16; ++k) tc::umma_bf16(d, da + k * 2, db + k * 128, id256, k > 0 ? 1u : acc0);
        }
        tc::umma_commit(&mi->o_done[g & 3]);
        cur.next(p.segs);
      }
    }
  } else {
    // ---------------- softmax / epilogue (warps 2-9) ----------------
    // Quadrant q of tensor memory holds heads 16q .. 16q+15.  The two warps of a quadrant split a
    // tile's 64 tokens; inside a warp, lanes 0-15 and 16-31 address the same 16 rows and split
    // the warp's 32 tokens again, so a thread owns 16 scores of one head.
    const int quad = warp & 3;
    const int half = (warp - 2) >> 2;
    const int sub = lane >> 4;
    const int row = quad * 16 + (lane & 15);
    const uint32_t lane_addr = tmem + ((uint32_t)(quad * 32) << 16);
    // epilogue staging: half of the P rows of this quadrant (what the two warps of the quadrant
    // write during the softmax, so the quadrant barrier orders the two uses)
    unsigned char* stage = s_stage + quad * 2048 + half * 1024;
    // The Q_eff block in ring slot gq -> tensor memory (bf16 pairs, two dims per column).  The block
    // came through the ring like a tile, ahead of the segment's first tile, so it does not queue
    // behind the tiles in flight as loads by these threads would.  Every QK MMA of the previous
    // segment must have retired (the caller saw s_full of its last tile).
    auto write_q = [&](int gq) -> bool {
      for (int i = 0; i < 3; ++i)
        if (!tc::mbar_wait(&mi->full_t[gq & 3][i], (gq >> 2) & 1, abort_flag, p.d_status, ST_SOFTMAX_TIMEOUT)) return false;
      const unsigned char* frame = s_ring + (gq % 3) * (NCH * CHUNK);
      // head `row`, dims 256*half + 128*gsel + 64*sub .. +63: row `row` of chunk 4*half + 2*gsel + sub
      // (128 bytes, eight 16-byte units, unit u at position u ^ (row & 7))
#pragma unroll
      for (int gsel = 0; gsel < 2; ++gsel) {
        const unsigned char* crow = frame + (half * 4 + gsel * 2 + sub) * CHUNK + row * 128;
        float w[32];
#pragma unroll
        for (int u = 0; u < 8; ++u) {
          const uint4 v = *reinterpret_cast<const uint4*>(crow + ((u ^ (row & 7)) * 16));
          w[u * 4] = __uint_as_float(v.x);
          w[u * 4 + 1] = __uint_as_float(v.y);
          w[u * 4 + 2] = __uint_as_float(v.z);
          w[u * 4 + 3] = __uint_as_float(v.w);
        }
        tmem_st16x64(lane_addr + COL_Q + half * 128 + gsel * 64, w);
      }
      if (NCH == 9 && half == 1) {  // the 64 rope dims (chunk 8): columns [256, 288)
        const unsigned char* crow = frame + 8 * CHUNK + row * 128;
        float w[16];
#pragma unroll
        for (int u = 0; u < 4; ++u) {
          const uint4 v = *reinterpret_cast<const uint4*>(crow + (((sub * 4 + u) ^ (row & 7)) * 16));
          w[u * 4] = __uint_as_float(v.x);
          w[u * 4 + 1] = __uint_as_float(v.y);
          w[u * 4 + 2] = __uint_as_float(v.z);
          w[u * 4 + 3] = __uint_as_float(v.w);
        }
        tmem_st16x32(lane_addr + COL_Q + 256, w);
      }
      tmem_wait_st();
      tc::tc_fence_before();
      tc::mbar_arrive(&mi->q_ready);
      return true;
    };
    TileCursor cur;
    cur.init(p.segs, seg0, seg1);
    bool ok = true;
    while (!cur.done() && ok) {
      const AttnSeg sg = cur.sg;
      const int n_tiles = cur.n_tiles;
      const unsigned span = (unsigned)(sg.kv_end - sg.kv_begin);
      // Q_eff of the first segment; later segments are written at the end of their predecessor
      if (cur.sidx == 0) ok = write_q(cur.gq);
      float m_used = -INFINITY, l = 0.0f;
      int g = cur.g;
      for (int t = 0; t < n_tiles && ok; ++t, cur.next(p.segs)) {
        g = cur.g;
        const int n = cur.n;
        ok = tc::mbar_wait(&mi->s_full[WHOLE ? n % 3 : n & 1], (WHOLE ? n / 3 : n >> 1) & 1, abort_flag, p.d_status, ST_SOFTMAX_TIMEOUT);
        tc::tc_fence_after();
        // this thread's first token, relative to the first visible row; visible: [0, span)
        const int rel0 = (sg.kv_begin & ~(TILE - 1)) - sg.kv_begin + t * TILE + half * 32 + sub * 16;
        float sc[16], sc2[16];
        const int b0 = WHOLE ? n % 3 : (2 * n) % 3, b1 = (2 * n + 1) % 3;
        tmem_ld16x32(lane_addr + COL_S + b0 * TILE + half * 32, sc);
        if (WHOLE) {
#pragma unroll
          for (int j = 0; j < 16; ++j) sc2[j] = 0.0f;
        } else {
          tmem_ld16x32(lane_addr + COL_S + b1 * TILE + half * 32, sc2);
        }
        tc::tc_fence_before();
        tc::mbar_arrive(&mi->s_free[b0]);
        if (!WHOLE) tc::mbar_arrive(&mi->s_free[b1]);
        float mx = -INFINITY;
#pragma unroll
        for (int j = 0; j < 16; ++j) {
          sc[j] = (unsigned)(rel0 + j) < span ? (sc[j] + sc2[j]) * p.scale_log2 : -INFINITY;
          mx = fmaxf(mx, sc[j]);
        }
        mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 16));
        if (sub == 0) mi->pmax[n & 1][half][row] = mx;
        ok = quad_bar_and(quad, ok);
        if (!ok) break;
        // the reference maximum moves only when the tile maximum exceeds it by more than 2^8
        const float tm = fmaxf(mi->pmax[n & 1][0][row], mi->pmax[n & 1][1][row]);
        float alpha = 1.0f;
        if (tm > m_used + RESCALE_THRESHOLD) {  // also the first tile (m_used = -inf)
          alpha = ex2f(m_used - tm);
          m_used = tm;
        }
        float sum = 0.0f;
        uint32_t packed[8];
#pragma unroll
        for (int j = 0; j < 16; j += 2) {
          const float p0 = ex2f(sc[j] - m_used), p1 = ex2f(sc[j + 1] - m_used);  // masked: ex2(-inf) = 0
          sum += p0 + p1;
          __nv_bfloat162 b = __floats2bfloat162_rn(p0, p1);
          packed[j / 2] = *reinterpret_cast<uint32_t*>(&b);
        }
        l = l * alpha + sum;
        // P (and O, if it is rescaled below) belong to the SV MMAs of the previous tile until they
        // retire (before a segment's first tile the epilogue has waited for them already)
        {
          // P[row, tokens 32*half + 16*sub .. +15]: two 16-byte units of the row, 128-byte swizzle.
          // The tile's own P buffer is free: with nine chunks it is the frame's rope chunk, which
          // the QK MMAs of this tile (retired: s_full) were the last to read; with eight it was last
          // read by the SV MMAs of the tile three slots back, which retired before this frame was
          // filled.
          unsigned char* prow = s_ring + p_slot_off<NCH>(g) + row * 128;
          const int u0 = half * 4 + sub * 2;
          *reinterpret_cast<uint4*>(prow + (((u0) ^ (row & 7)) * 16)) = make_uint4(packed[0], packed[1], packed[2], packed[3]);
          *reinterpret_cast<uint4*>(prow + (((u0 + 1) ^ (row & 7)) * 16)) = make_uint4(packed[4], packed[5], packed[6], packed[7]);
        }
        // O rows are scaled by their own alpha through the 16-lane access shape at lane offset 16
        // (O belongs to the SV MMAs of the previous tile until they retire: only this path waits)
        if (t > 0 && __any_sync(0xffffffffu, alpha != 1.0f)) {
          ok = tc::mbar_wait(&mi->o_done[(g - 1) & 3], ((g - 1) >> 2) & 1, abort_flag, p.d_status, ST_SOFTMAX_TIMEOUT);
          ok = __all_sync(0xffffffffu, ok);  // (the tensor-memory accesses below are warp-collective)
          if (!ok) break;
          tc::tc_fence_after();
#pragma unroll 1
          for (int cc = 0; cc < 4; ++cc) {
            float o[32];
            const uint32_t addr = lane_addr + LANE16 + COL_O + half * 256 + cc * 64;
            tmem_ld16x64(addr, o);
#pragma unroll
            for (int j = 0; j < 32; ++j) o[j] *= alpha;
            tmem_st16x64(addr, o);
          }
          tmem_wait_st();
        }
        tc::fence_proxy_async();
        tc::tc_fence_before();
        tc::mbar_arrive(&mi->p_full[n % 3]);
      }
      if (!ok) break;
      // Q_eff of the next segment goes in first, so that its QK MMAs run during the epilogue
      if (!cur.done()) ok = write_q(cur.gq);
      if (!ok) break;
      // ---- epilogue of the segment: un-normalised partial (max, sum, O) ----
      ok = tc::mbar_wait(&mi->o_done[g & 3], (g >> 2) & 1, abort_flag, p.d_status, ST_EPI_TIMEOUT);
      tc::tc_fence_after();
      l += __shfl_xor_sync(0xffffffffu, l, 16);
      if (sub == 0) mi->lsum[half][row] = l;
      ok = quad_bar_and(quad, ok);
      if (!ok) break;
      if (DIRECT && p.tok_part[sg.tok + 1] - p.tok_part[sg.tok] == 1) {
        finish_token(p, sg.tok, row, half, sub, lane_addr, m_used * 0.6931471805599453f,
                     mi->lsum[0][row] + mi->lsum[1][row]);
      } else {
        if (half == 0 && sub == 0) {
          p.part_l[(long long)sg.part * HEADS + row] = mi->lsum[0][row] + mi->lsum[1][row];
          p.part_m[(long long)sg.part * HEADS + row] = m_used * 0.6931471805599453f;  // back to ln units
        }
        {
          // A 32-lane load hands lanes 16-31 the O rows of this quadrant (row lane-16), 32 columns
          // at a time; this warp owns columns 256*half .. +255.  The rows go through shared memory
          // so that every store instruction writes four full 128-byte lines.
          float* po = p.part_o + ((long long)sg.part * HEADS + quad * 16) * D_V + half * 256;
          if (cur.done()) {
            // The CTA's last segment: every tile has retired, so the ring is idle and each warp
            // stages its whole 16 x 256 block there (16 KB) -- all tensor-memory loads first, one
            // warp barrier, then the stores back to back instead of 16 small round trips.
            unsigned char* big = s_ring + (warp - 2) * 16384;
#pragma unroll 1
            for (int cc = 0; cc < 8; ++cc) {
              float o[32];
              tc::tmem_ld32(lane_addr + COL_O + half * 256 + cc * 32, o);
              if (sub == 1) {
                const int rr = lane - 16;
#pragma unroll
                for (int u = 0; u < 8; ++u)
                  *reinterpret_cast<float4*>(big + cc * 2048 + rr * 128 + ((u ^ (rr & 7)) * 16)) =
                      make_float4(o[u * 4], o[u * 4 + 1], o[u * 4 + 2], o[u * 4 + 3]);
              }
            }
            __syncwarp();
#pragma unroll 4
            for (int i = 0; i < 32; ++i) {
              const int cc = i >> 2, rr = (i & 3) * 4 + (lane >> 3), u = lane & 7;
              const float4 v = *reinterpret_cast<const float4*>(big + cc * 2048 + rr * 128 + ((u ^ (rr & 7)) * 16));
              *reinterpret_cast<float4*>(po + (long long)rr * D_V + cc * 32 + u * 4) = v;
            }
          } else {
#pragma unroll 1
            for (int cc = 0; cc < 8; ++cc) {
              float o[32];
              tc::tmem_ld32(lane_addr + COL_O + half * 256 + cc * 32, o);
#pragma unroll
              for (int h8 = 0; h8 < 2; ++h8) {  // eight rows at a time through the 1 KB staging area
                if (sub == 1 && ((lane >> 3) & 1) == h8) {
                  const int rr = lane & 7;
#pragma unroll
                  for (int u = 0; u < 8; ++u)
                    *reinterpret_cast<float4*>(stage + rr * 128 + ((u ^ rr) * 16)) = make_float4(o[u * 4], o[u * 4 + 1], o[u * 4 + 2], o[u * 4 + 3]);
                }
                __syncwarp();
#pragma unroll
                for (int i = 0; i < 2; ++i) {
                  const int rr = i * 4 + (lane >> 3), u = lane & 7;
                  const float4 v = *reinterpret_cast<const float4*>(stage + rr * 128 + ((u ^ rr) * 16));
                  *reinterpret_cast<float4*>(po + (long long)(h8 * 8 + rr) * D_V + cc * 32 + u * 4) = v;
                }
                __syncwarp();
              }
            }
          }
        }
      }
      tc::tc_fence_before();
      ok = quad_bar_and(quad, ok);  // lsum, the staging rows and O are reused by the next segment
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
  __syncthreads();
}

}  // namespace


bool attn_stream_supported(const AttnArgs& a) {
  return a.H == HEADS && a.d_v == D_V && a.page_tokens == TILE && a.row == a.d_qk &&
         (a.d_qk == 576 || a.d_qk == 512) && a.pool_rows < (1ll << 31) &&
         (reinterpret_cast<uintptr_t>(a.pool) & 15) == 0 && (reinterpret_cast<uintptr_t>(a.q_eff) & 15) == 0;
}

cudaError_t launch_attn_stream(const AttnArgs& a, cudaStream_t st) {
  static_assert(sizeof(StreamMisc) <= MISC_BYTES, "misc region too small");
  static_assert(smem_total(9) <= 227 * 1024 && smem_total(8) <= 227 * 1024, "shared memory budget");
  static_assert(COL_S + 3 * TILE <= TMEM_COLS, "tensor memory budget");
  if (a.n_segs <= 0) return cudaSuccess;
  CUtensorMap tmKV;
  const char* err = nullptr;
  if (!tc::cached_tmap(&tmKV, a.pool, (uint64_t)a.row, (uint64_t)a.pool_rows, 1, (uint64_t)a.row * 2,
                       (uint64_t)a.row * 2 * (uint64_t)a.pool_rows, 64, TILE, 1, &err))
    return cudaErrorInvalidValue;
  // Q_eff has the geometry of the pool: rows of d_qk values, a token's 64 heads are one "page"
  CUtensorMap tmQ;
  if (!tc::cached_tmap(&tmQ, a.q_eff, (uint64_t)a.d_qk, (uint64_t)a.q_rows, 1, (uint64_t)a.d_qk * 2,
                       (uint64_t)a.d_qk * 2 * (uint64_t)a.q_rows, 64, HEADS, 1, &err))
    return cudaErrorInvalidValue;
  StreamParams p;
  p.q_eff = a.q_eff; p.tables = a.tables; p.segs = a.segs; p.cta_seg = a.cta_seg;
  p.part_m = a.part_m; p.part_l = a.part_l; p.part_o = a.part_o; p.d_status = a.d_status;
  p.pool = a.pool;
  p.d_qk = a.d_qk;
  p.scale_log2 = a.scale * 1.4426950408889634f;
  p.direct = a.direct_single ? 1 : 0;
  p.tok_part = a.tok_part; p.o_lat = a.o_lat; p.sinks = a.sinks; p.lut = a.lut;
  p.rope = a.rope; p.inv_rope = a.inv_rope;
  p.tiles_shared = a.tiles_shared ? 1 : 0;
  const bool whole = a.tiles_shared;
#define FST_ATTN_LAUNCH(NCHV, DIR, WH) \
  launch_k(a.dependent_launch, k_attn_stream<NCHV, DIR, WH>, dim3(a.n_ctas), dim3(ST_THREADS), smem_total(NCHV), st, 1, tmKV, tmQ, p)
  if (a.d_qk == 576) {
    if (whole) return p.direct ? FST_ATTN_LAUNCH(9, true, true) : FST_ATTN_LAUNCH(9, false, true);
    return p.direct ? FST_ATTN_LAUNCH(9, true, false) : FST_ATTN_LAUNCH(9, false, false);
  }
  if (whole) return p.direct ? FST_ATTN_LAUNCH(8, true, true) : FST_ATTN_LAUNCH(8, false, true);
  return p.direct ? FST_ATTN_LAUNCH(8, true, false) : FST_ATTN_LAUNCH(8, false, false);
#undef FST_ATTN_LAUNCH
}

}  // namespace fst
