// Shared device helpers for the sm_100a MLA kernels.
#pragma once
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>

namespace fst {

typedef __nv_bfloat16 bf16;

__device__ __forceinline__ float bf2f(bf16 v) { return __bfloat162float(v); }
__device__ __forceinline__ bf16 f2bf(float v) { return __float2bfloat16_rn(v); }
// Round-trip through bf16 (round-to-nearest-even), where the reference stores a bf16 buffer.
__device__ __forceinline__ float rbf(float v) { return bf2f(f2bf(v)); }

__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  return v;
}
__device__ __forceinline__ float warp_max(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
  return v;
}

// Sum over a block of up to 1024 threads; `scratch` holds 32 floats. All threads get the sum.
__device__ __forceinline__ float block_sum(float v, float* scratch) {
  const int lane = threadIdx.x & 31, wid = threadIdx.x >> 5, nw = (blockDim.x + 31) >> 5;
  v = warp_sum(v);
  __syncthreads();
  if (lane == 0) scratch[wid] = v;
  __syncthreads();
  float t = lane < nw ? scratch[lane] : 0.0f;
  return warp_sum(t);
}

// Programmatic dependent launch: the kernels of a layer call are launched with programmatic
// stream serialisation, so a kernel's prologue (barrier set-up, TMEM allocation, loads of
// weights, which no earlier kernel writes) runs while its predecessor drains.  pdl_launch lets
// the successor start; pdl_wait blocks until every earlier kernel has completed and its writes
// are visible -- every thread calls it before it touches anything an earlier kernel produced.
__device__ __forceinline__ void pdl_launch() { asm volatile("griddepcontrol.launch_dependents;" ::: "memory"); }
__device__ __forceinline__ void pdl_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }


// One segment of the split-KV schedule: query token `tok` attends to rows [kv_begin, kv_end) of
// the row space whose block table starts at entry `table` of the flat table array -- the raw rows
// of its sequence, or (layers with a KV compressor) the compressed rows, which live in pages of
// their own -- and writes partial slot `part`.
struct AttnSeg {
  int32_t tok;
  int32_t kv_begin;
  int32_t kv_end;
  int32_t part;
  int32_t table;
};

// Status word values written by kernels that give up a bounded wait.
enum : int { ST_OK = 0, ST_TMA_TIMEOUT = 1, ST_MMA_TIMEOUT = 2, ST_SOFTMAX_TIMEOUT = 3, ST_EPI_TIMEOUT = 4,
              ST_SELFTEST_TIMEOUT = 5 };

}  // namespace fst
