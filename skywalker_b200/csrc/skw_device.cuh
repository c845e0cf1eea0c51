// Device-side arithmetic shared by every kernel of the library: the Philox4x32-10 stream, the
// mapping from random words to columns / uniforms, the alias slot, and the per-launch error word.
#pragma once
#include <cuda_runtime.h>
#include <stdint.h>

namespace skw {

typedef uint32_t u32;
typedef uint64_t u64;

// One entry of the alias table: keep column i with probability prob, else take column alias.
// 8 bytes so that a draw costs one vectorised load (the reference keeps two arrays,
// gpu_graph::prob_array / alias_array, include/gpu_graph.cuh:40-60, i.e. two sectors per draw).
struct __align__(8) Slot {
  float prob;
  u32 alias;
};

// Purpose tags xor-ed into the high key word so that streams of different uses never overlap.
enum : u32 {
  TAG_WALK = 0x57414C4Bu, TAG_KHOP = 0x4B484F50u, TAG_RMAT = 0x524D4154u,
  TAG_WGHT = 0x57474854u, TAG_STRT = 0x53545254u, TAG_PLAW = 0x504C4157u
};

struct Rand4 {
  u32 x, y, z, w;
};

// Philox4x32-10 (Salmon et al., SC'11): counter (c0..c3), key (k0,k1).
__device__ __forceinline__ Rand4 philox4x32_10(u32 c0, u32 c1, u32 c2, u32 c3, u32 k0, u32 k1) {
#pragma unroll
  for (int r = 0; r < 10; ++r) {
    const u32 hi0 = __umulhi(0xD2511F53u, c0), lo0 = 0xD2511F53u * c0;
    const u32 hi1 = __umulhi(0xCD9E8D57u, c2), lo1 = 0xCD9E8D57u * c2;
    c0 = hi1 ^ c1 ^ k0;
    c1 = lo1;
    c2 = hi0 ^ c3 ^ k1;
    c3 = lo0;
    k0 += 0x9E3779B9u;
    k1 += 0xBB67AE85u;
  }
  return Rand4{c0, c1, c2, c3};
}
__device__ __forceinline__ Rand4 philox_tagged(u64 seed, u32 tag, u64 unit, u32 c2, u32 c3) {
  return philox4x32_10((u32)unit, (u32)(unit >> 32), c2, c3, (u32)seed, (u32)(seed >> 32) ^ tag);
}
// 24-bit uniform in [0,1); exact in fp32.
__device__ __forceinline__ float u01(u32 r) { return (float)(r >> 8) * 5.9604644775390625e-8f; }

// Error word written by kernels instead of trapping: err[0] = first code, err[1..3] = detail.
enum : u32 {
  DEV_OK = 0,
  DEV_ERR_INDEX = 1,     // an index left its array
  DEV_ERR_WAIT = 2,      // a bounded wait ran out
  DEV_ERR_CAPACITY = 3,  // a work list or scratch slab was too small
  DEV_ERR_INTERNAL = 4   // an invariant of the construction did not hold
};
__device__ __forceinline__ void dev_fail(u32* err, u32 code, u32 a, u32 b, u32 c) {
  if (atomicCAS(err, 0u, code) == 0u) {
    err[1] = a;
    err[2] = b;
    err[3] = c;
  }
}

// Read-only loads for data that is touched at random and used once.  A plain load that misses L1
// pulls the whole 128-byte line from DRAM; these ask for the smallest L2 fetch (64 bytes) and do
// not allocate in L1.  Same access rate on B200, half the DRAM traffic.
__device__ __forceinline__ u32 ldg_once(const u32* p) {
  u32 v;
  asm volatile("ld.global.nc.L1::no_allocate.L2::64B.u32 %0, [%1];" : "=r"(v) : "l"(p));
  return v;
}
__device__ __forceinline__ uint2 ldg_once(const uint2* p) {
  uint2 v;
  asm volatile("ld.global.nc.L1::no_allocate.L2::64B.v2.u32 {%0,%1}, [%2];" : "=r"(v.x), "=r"(v.y) : "l"(p));
  return v;
}

__device__ __forceinline__ Slot load_slot(const Slot* p) {
  const uint2 v = ldg_once(reinterpret_cast<const uint2*>(p));
  Slot s;
  s.prob = __uint_as_float(v.x);
  s.alias = v.y;
  return s;
}

}  // namespace skw
