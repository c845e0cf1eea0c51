// Shared by the walk kernels: launch arguments, the connectivity test of node2vec, the edge counter.
#pragma once
#include "skw_ctx.h"

namespace skw {

constexpr u32 kAlive = 0xFFFFFFFFu;
constexpr u32 kNoVertex = 0xFFFFFFFFu;
constexpr u32 kN2vMaxTrials = 64;

struct WalkArgs {
  const u32* xadj;
  const u32* adjncy;
  const Slot* slots;
  const u32* starts;
  u32* paths;
  u32* lengths;
  unsigned long long* sum;
  u32* err;
  u64 n;
  u64 seed;
  u64 walker_base;
  u64 walker_stride;
  u32 V;
  u32 hop_num;
  u32 unbiased;  // uniform neighbour choice: no table is read
  float tp, inv_p, inv_q, fmax;
};

// bool CheckConnect(src, dst) of the reference (include/gpu_graph.cuh:204-238): binary search of
// dst in the sorted adjacency of src.
__device__ __forceinline__ bool connected(const u32* __restrict__ xadj,
                                          const u32* __restrict__ adjncy, u32 src, u32 dst) {
  u32 lo = __ldg(xadj + src), hi = __ldg(xadj + src + 1);
  while (lo < hi) {
    const u32 mid = lo + ((hi - lo) >> 1);
    const u32 x = __ldg(adjncy + mid);
    if (x == dst) return true;
    if (x < dst) lo = mid + 1;
    else hi = mid;
  }
  return false;
}

__device__ __forceinline__ void add_edges(unsigned long long* sum, u64 edges) {
#pragma unroll
  for (int o = 16; o; o >>= 1) edges += __shfl_xor_sync(0xFFFFFFFFu, edges, o);
  if ((threadIdx.x & 31) == 0 && edges) atomicAdd(sum, (unsigned long long)edges);
}

// One warp per walker, every step's slot computed from the weight list (skw_walk_direct.cu).
int launch_walk_online_direct(skw_ctx* ctx, const WalkArgs& a, uint32_t app);

}  // namespace skw
