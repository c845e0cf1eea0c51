// Offline alias-table construction for all vertices of a range.
//
// Takes over ConstructTable / ConstructAliasTableKernel (src/createTable.cu:48-179 of the
// reference) and the alias_table_constructor_shmem methods it drives (loadFromGraph, construct,
// constructBC, SaveAliasTable; include/alias_table_new.cuh:1077-1132, 1211-1316, 334-464,
// 1105-1115).
//
// Construction rule (one vertex, degree n, weights w_0..w_{n-1}; identical to the sequential
// sweep "smalls in index order are topped up by larges in index order, a large that falls below
// one bucket is topped up by the next large"):
//   masses    B = min(40, 62 - ceil(log2 n)), C = 2^B, q_i = trunc(w_i * 2^(B-1-e)) with
//             e = floor(log2 max w), Q_i = q_0 + .. + q_(i-1), W = Q_n, K = n*C / W (one IEEE
//             double division), g(Q) = n*C if Q == W else min(n*C, trunc((double)Q * K)),
//             M_i = g(Q_i + q_i) - g(Q_i).  g is monotone, so zero weights get zero mass and
//             sum M_i == n*C exactly.
//   classes   small: M_i < C, large: M_i >= C.
//   prefixes  D(i) = sum over smalls at positions <= i of (C - M), X(i) = sum over larges at
//             positions <= i of (M - C)   (both over list positions, zeros elsewhere).
//   small s   alias = first large l at or after the first position with X >= D(s) - (C - M_s),
//             prob  = M_s / C.
//   large l   let S = first position with D(S) > X(l); if none: prob = 1, alias = l; else
//             prob = (X(l) + C - D(S)) / C, alias = next large after l.
// Every quantity is an integer or a single correctly rounded IEEE operation, so the table is a
// pure function of the weight list: no atomics on masses, no dependence on scheduling.
//
// Work distribution: vertices are binned by degree into nine classes with warp ballots and
// shared-memory prefix sums (classify_* kernels); classes of degree <= 32 run one sub-warp
// group of 4/8/16/32 lanes per vertex entirely in registers; degree <= 256 and <= 1024 one warp
// per vertex, degree <= 4096 one CTA of 256 threads and degree <= 16384 one CTA of 1024 threads per
// vertex, with the two prefix lists in shared memory; larger vertices one CTA of 1024 threads with
// the lists in a global scratch slab, merged through shared-memory windows.
#include <math_constants.h>

#include <cstdarg>
#include <cstdio>
#include <mutex>

#include "skw_alias_math.cuh"
#include "skw_ctx.h"

namespace skw {

// degree classes: groups of 4/8/16/32 lanes; one warp per vertex (two capacities); one CTA of
// 256 threads with its lists in shared memory; one CTA of 1024 threads with its lists in a
// global scratch slab, merged through shared-memory windows
enum { K_G1 = 0, K_G2, K_G4, K_G8, K_G16, K_G32, K_W1K, K_C, K_C2A, K_C2, K_H, K_CLASSES };
constexpr u32 kGroupEpt = 8;          // list elements a lane of a sub-warp group keeps in registers
constexpr u32 kWarpSmallMax = 32 * kGroupEpt;  // 256: the largest list a whole warp holds in registers
constexpr u32 kWarpMax = 1024;
constexpr u32 kLargeMax = kCtaSmemMaxDegree;  // 4096: 12 bytes of list state per edge, 4 CTAs per SM
constexpr u32 kMidSmemMax = 8192;             // two 512-thread CTAs per SM with 96 KB of lists each
constexpr u32 kHugeSmemMax = 16384;           // one 1024-thread CTA per SM with 192 KB of lists

__device__ __forceinline__ int degree_class(u32 deg) {
  if (deg <= kWarpSmallMax) {  // groups of 1, 2, 4 ... 32 lanes, kGroupEpt elements per lane
    if (deg <= kGroupEpt) return K_G1;
    return K_G1 + (32 - __clz((int)((deg - 1) / kGroupEpt)));
  }
  if (deg <= kWarpMax) return K_W1K;
  if (deg <= kLargeMax) return K_C;
  if (deg <= kMidSmemMax) return K_C2A;
  if (deg <= kHugeSmemMax) return K_C2;
  return K_H;
}

// cls[0..K) counts, cls[K..2K) fill cursors, cls[2K..3K) bases of the classes in the work list,
// cls[3K..4K) cursors from which the builder kernels take their next vertex.
__global__ void __launch_bounds__(256) classify_count_kernel(const u32* __restrict__ xadj,
                                                             u32 v_begin, u32 v_end,
                                                             u32* __restrict__ cls,
                                                             uint8_t* __restrict__ valid) {
  __shared__ u32 s_cnt[K_CLASSES];
  if (threadIdx.x < K_CLASSES) s_cnt[threadIdx.x] = 0;
  __syncthreads();
  const u32 lane = threadIdx.x & 31;
  for (u64 v0 = v_begin + (u64)blockIdx.x * blockDim.x; v0 < v_end; v0 += (u64)gridDim.x * blockDim.x) {
    const u64 v = v0 + threadIdx.x;
    int c = -1;
    if (v < v_end) {
      const u32 deg = xadj[v + 1] - xadj[v];
      if (deg == 0) valid[v] = 0;
      else c = degree_class(deg);
    }
#pragma unroll
    for (int k = 0; k < K_CLASSES; ++k) {
      const u32 m = __ballot_sync(0xFFFFFFFFu, c == k);
      if (lane == 0 && m) atomicAdd(&s_cnt[k], __popc(m));
    }
  }
  __syncthreads();
  if (threadIdx.x < K_CLASSES && s_cnt[threadIdx.x]) atomicAdd(&cls[threadIdx.x], s_cnt[threadIdx.x]);
}

__global__ void classify_bases_kernel(u32* __restrict__ cls) {
  if (threadIdx.x == 0) {
    u32 run = 0;
    for (int k = 0; k < K_CLASSES; ++k) {
      cls[2 * K_CLASSES + k] = run;
      cls[K_CLASSES + k] = 0;
      run += cls[k];
    }
  }
}

// Ordered compaction inside a block (ballot + shared prefix), one atomic per class per block
// tile to reserve the output range.
__global__ void __launch_bounds__(256) classify_fill_kernel(const u32* __restrict__ xadj,
                                                            u32 v_begin, u32 v_end,
                                                            u32* __restrict__ cls,
                                                            u32* __restrict__ worklist) {
  __shared__ u32 s_warp[K_CLASSES][8];
  __shared__ u32 s_base[K_CLASSES];
  const u32 lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  for (u64 v0 = v_begin + (u64)blockIdx.x * blockDim.x; v0 < v_end; v0 += (u64)gridDim.x * blockDim.x) {
    const u64 v = v0 + threadIdx.x;
    int c = -1;
    if (v < v_end) {
      const u32 deg = xadj[v + 1] - xadj[v];
      if (deg) c = degree_class(deg);
    }
    u32 my_rank = 0;
#pragma unroll
    for (int k = 0; k < K_CLASSES; ++k) {
      const u32 m = __ballot_sync(0xFFFFFFFFu, c == k);
      if (c == k) my_rank = __popc(m & ((1u << lane) - 1u));
      if (lane == 0) s_warp[k][warp] = __popc(m);
    }
    __syncthreads();
    if (threadIdx.x < K_CLASSES) {
      u32 run = 0;
      for (int w = 0; w < 8; ++w) {
        const u32 t = s_warp[threadIdx.x][w];
        s_warp[threadIdx.x][w] = run;
        run += t;
      }
      s_base[threadIdx.x] =
          run ? cls[2 * K_CLASSES + threadIdx.x] + atomicAdd(&cls[K_CLASSES + threadIdx.x], run) : 0;
    }
    __syncthreads();
    if (c >= 0) worklist[s_base[c] + s_warp[c][warp] + my_rank] = (u32)v;
    __syncthreads();
  }
}

// ------------------------------------------------------------------ bulk copy (TMA unit) ---
// Untiled cp.async.bulk global -> shared with completion on an mbarrier.  Both addresses must be
// 16-byte aligned and the size a multiple of 16 bytes; the caller rounds the window inwards and
// fetches ragged ends with plain loads.  No multicast, local memory only.
__device__ __forceinline__ u32 smem_addr(const void* p) { return (u32)__cvta_generic_to_shared(p); }
__device__ __forceinline__ void mbar_init(u64* bar, u32 arrivals) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_addr(bar)), "r"(arrivals) : "memory");
  asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
}
__device__ __forceinline__ void bulk_copy_g2s(void* dst, const void* src, u32 bytes, u64* bar) {
  // order earlier generic-proxy accesses of the destination before the async-proxy writes
  asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(smem_addr(bar)), "r"(bytes) : "memory");
  asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::"r"(
                   smem_addr(dst)),
               "l"(src), "r"(bytes), "r"(smem_addr(bar))
               : "memory");
}
// One arrival without bytes to wait for (a phase that no bulk copy feeds).
__device__ __forceinline__ void mbar_arrive(u64* bar) {
  asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(smem_addr(bar)) : "memory");
}
// Poll (without blocking) for the phase with the given parity, at most `limit` times with a short
// sleep in between: a few milliseconds in total.  Returns false if the copy did not complete.
__device__ __forceinline__ bool mbar_wait(u64* bar, u32 parity, u32 limit) {
  for (u32 i = 0; i < limit; ++i) {
    u32 done;
    asm volatile(
        "{\n\t.reg .pred p;\n\tmbarrier.test_wait.parity.shared::cta.b64 p, [%1], %2;\n\tselp.u32 %0, 1, 0, p;\n\t}"
        : "=r"(done)
        : "r"(smem_addr(bar)), "r"(parity)
        : "memory");
    if (done) return true;
    __nanosleep(32);
  }
  return false;
}

// ------------------------------------------------------------------ merge-path builders ----
// NT cooperating threads (one warp, or a CTA) build one vertex.
//
// The sweep "smalls in index order are topped up by larges in index order" is a MERGE of two
// sorted lists: small i (key = deficit of the smalls before it) comes before large j (key = excess
// of the larges up to and including it) iff its key is <= the large's key.  When small i is
// emitted at state (i, j) its donor is large j; when large j is emitted while smalls remain it
// has fallen below one bucket, keeps X(j) + C - D(i-1) of it and is topped up by large j+1; larges
// emitted after the last small own exactly one bucket.  So after the two prefix lists are in
// memory, every thread takes an equal slice of the merged order (merge-path partition by one
// bisection per thread) and runs the sweep serially on it: the same number of steps in every
// lane, no per-element searches.
//
// Phase 1 walks the weight list in tiles of NT*4 elements (4 consecutive elements per thread, so a
// prefix sum is a short serial scan plus one cross-thread scan) and writes
//   A[i] = inclusive deficit prefix of small i,   P[i] = its position        (smalls from the front)
//   A[n-1-j] = inclusive excess prefix of large j, P[n-1-j] = its position   (larges from the back)
template <int NT>
__device__ __forceinline__ void coop_sync() {
  if constexpr (NT == 32) __syncwarp();
  else __syncthreads();
}

// Exclusive cross-thread prefix and total of one u64 per thread.  In a CTA the warp totals are
// scanned by the first warp (s_tmp: NT/32 + 1 entries).
template <int NT>
__device__ __forceinline__ void coop_scan_u64(u64& v, u64& total, u64* s_tmp) {
  const u32 lane = threadIdx.x & 31;
  u64 inc = v;
#pragma unroll
  for (int o = 1; o < 32; o <<= 1) {
    const u64 t = __shfl_up_sync(0xFFFFFFFFu, inc, o);
    if (lane >= (u32)o) inc += t;
  }
  if constexpr (NT == 32) {
    total = __shfl_sync(0xFFFFFFFFu, inc, 31);
    v = inc - v;
  } else {
    constexpr int NW = NT / 32;
    const u32 warp = threadIdx.x >> 5;
    __syncthreads();
    if (lane == 31) s_tmp[warp] = inc;
    __syncthreads();
    if (warp == 0) {
      u64 x = lane < NW ? s_tmp[lane] : 0, xi = x;
#pragma unroll
      for (int o = 1; o < 32; o <<= 1) {
        const u64 t = __shfl_up_sync(0xFFFFFFFFu, xi, o);
        if (lane >= (u32)o) xi += t;
      }
      if (lane < NW) s_tmp[lane] = xi - x;
      if (lane == 31) s_tmp[NW] = xi;
    }
    __syncthreads();
    total = s_tmp[NW];
    v = s_tmp[warp] + inc - v;
  }
}

// The same for a 64-bit and a 32-bit value at once (s_tmp: 2 * (NT/32 + 1) entries).
template <int NT>
__device__ __forceinline__ void coop_scan2(u64& a, u32& c, u64& ta, u32& tc, u64* s_tmp) {
  const u32 lane = threadIdx.x & 31;
  u64 ia = a;
  u32 ic = c;
#pragma unroll
  for (int o = 1; o < 32; o <<= 1) {
    const u64 xa = __shfl_up_sync(0xFFFFFFFFu, ia, o);
    const u32 xc = __shfl_up_sync(0xFFFFFFFFu, ic, o);
    if (lane >= (u32)o) {
      ia += xa;
      ic += xc;
    }
  }
  if constexpr (NT == 32) {
    ta = __shfl_sync(0xFFFFFFFFu, ia, 31);
    tc = __shfl_sync(0xFFFFFFFFu, ic, 31);
    a = ia - a;
    c = ic - c;
  } else {
    constexpr int NW = NT / 32, ST = NW + 1;
    const u32 warp = threadIdx.x >> 5;
    __syncthreads();
    if (lane == 31) {
      s_tmp[warp] = ia;
      s_tmp[ST + warp] = ic;
    }
    __syncthreads();
    if (warp == 0) {
      u64 xa = lane < NW ? s_tmp[lane] : 0;
      u32 xc = lane < NW ? (u32)s_tmp[ST + lane] : 0;
      u64 ya = xa;
      u32 yc = xc;
#pragma unroll
      for (int o = 1; o < 32; o <<= 1) {
        const u64 pa = __shfl_up_sync(0xFFFFFFFFu, ya, o);
        const u32 pc = __shfl_up_sync(0xFFFFFFFFu, yc, o);
        if (lane >= (u32)o) {
          ya += pa;
          yc += pc;
        }
      }
      if (lane < NW) {
        s_tmp[lane] = ya - xa;
        s_tmp[ST + lane] = yc - xc;
      }
      if (lane == 31) {
        s_tmp[NW] = ya;
        s_tmp[ST + NW] = yc;
      }
    }
    __syncthreads();
    ta = s_tmp[NW];
    tc = (u32)s_tmp[ST + NW];
    a = s_tmp[warp] + ia - a;
    c = (u32)s_tmp[ST + warp] + ic - c;
  }
}

template <int NT>
__device__ __forceinline__ float coop_max(float v, float* s_tmp) {
#pragma unroll
  for (int o = 16; o; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xFFFFFFFFu, v, o));
  if constexpr (NT != 32) {
    __syncthreads();
    if ((threadIdx.x & 31) == 0) s_tmp[threadIdx.x >> 5] = v;
    __syncthreads();
    float t = 0.0f;
#pragma unroll
    for (int w = 0; w < NT / 32; ++w) t = fmaxf(t, s_tmp[w]);
    v = t;
  }
  return v;
}

// Merge phase over one window: nl = Sl + Ll list entries (Sl smalls in sA[0..Sl), Ll larges from
// the back: large j' at nl-1-j'), positions in sP alike.  dsx_in = deficit of all smalls before
// the window, next_pos = position of the first large after the window (kNoNext if none).  Thread
// t emits an equal share of the window's merged order.
constexpr u32 kNoNext = 0xFFFFFFFFu;
template <int NT>
__device__ __forceinline__ void merge_window(u32 t, u32 nl, u32 Sl, const u64* sA, const u32* sP, u64 dsx_in,
                                             u32 next_pos, u64 C, int B, u32 off, Slot* __restrict__ slots,
                                             u32 v, u32* err) {
  const u32 Ll = nl - Sl;
  const u32 VT = (nl + NT - 1) / NT;
  const u32 k0 = min(t * VT, nl), k1 = min(k0 + VT, nl);
  if (k0 >= k1) return;
  u32 i, j;
  {
    u32 lo = k0 > Ll ? k0 - Ll : 0, hi = min(k0, Sl);
    while (lo < hi) {
      const u32 mid = (lo + hi) >> 1;
      const u64 a = mid ? sA[mid - 1] : dsx_in;    // key of small mid
      const u64 b = sA[nl - 1 - (k0 - 1 - mid)];   // key of large k0-1-mid
      if (a <= b) lo = mid + 1;
      else hi = mid;
    }
    i = lo;
    j = k0 - lo;
  }
  // i <= Sl and j <= Ll hold from here on, and i + j = k < nl: the entry that leaves always exists.
  // A step has no branch (see merge_packed): a window of three entries stays in registers, the
  // small at the head, the large at the head and the large behind it; past the window's last large
  // the key is "never full" and the position that of the next window's first large.
  constexpr u64 kNever = ~0ull;
  u64 dsx = i ? sA[i - 1] : dsx_in;  // deficit of the smalls before small i
  u64 sk = 0, lk = kNever, lk2 = kNever;
  u32 sp = 0, lp = next_pos, lp2 = next_pos;
  if (i < Sl) {
    sk = sA[i];
    sp = sP[i];
  }
  if (j < Ll) {
    lk = sA[nl - 1 - j];
    lp = sP[nl - 1 - j];
  }
  if (j + 1 < Ll) {
    lk2 = sA[nl - 2 - j];
    lp2 = sP[nl - 2 - j];
  }
  Slot* __restrict__ out = slots + off;
  bool bad = false;
  for (u32 k = k0; k < k1; ++k) {
    const bool fits = dsx <= lk;
    const bool take = i < Sl && fits;              // a small leaves; else a large
    const bool full = !take && fits;               // only once every small is placed
    const u32 p = take ? sp : lp;
    const u32 a = take ? lp : lp2;                 // a small's alias: the large at the head; a large's: the next one
    const bool none = a == kNoNext;
    bad |= none && !full;                          // mass conservation rules it out
    const bool self = full || none;
    const u64 x = take ? dsx : lk, y = take ? sk : dsx;  // small: C - (sk - dsx); large: lk + C - dsx
    Slot o;
    o.prob = self ? 1.0f : mass_to_prob_fast(C + x - y, B);
    o.alias = self ? p : a;
    out[p] = o;
    i += take ? 1u : 0u;
    j += take ? 0u : 1u;
    const u32 idx = take ? i : nl - 2 - j;
    const bool more = take ? i < Sl : j + 1 < Ll;
    const u64 nk = more ? sA[idx] : kNever;
    const u32 np = more ? sP[idx] : next_pos;
    dsx = take ? sk : dsx;
    lk = take ? lk : lk2;
    lp = take ? lp : lp2;
    lk2 = take ? lk2 : nk;
    lp2 = take ? lp2 : np;
    sk = take ? nk : sk;
    sp = take ? np : sp;
  }
  if (bad) dev_fail(err, DEV_ERR_INTERNAL, v, k0, 8);
}

// WIN == 0: the lists A / P are in shared memory and are merged in place.  WIN > 0: they are in
// global scratch and win_smem holds WIN * 12 + (NT + 1) * 4 bytes of shared memory for staging.
// NBUF > 0: the tiles of the weight list come through `pipe` (see TilePipe) instead of global loads, with
// two buffers one tile ahead of the one being worked on, with one buffer refilled as soon as a tile's
// weights are quantised.
// STAGED: w points at a copy of the weight list in shared memory, else at the list in global memory.
// Weight tiles of the scratch class brought into shared memory by the bulk-copy engine, one tile
// ahead of the one being worked on: two buffers of tile + 8 floats and one mbarrier each.  The parity
// of each barrier's current phase lives in `parity` (bit b for buffer b) across the vertices of a CTA.
struct TilePipe {
  float* buf;   // 2 x (tile + 8) floats, 16-byte aligned
  u64* bars;    // 2 mbarriers, initialised with one arrival
  u32 parity;
  bool failed;  // a copy did not report completion in time: the CTA stops taking vertices
};

template <int NT, int EPT, int WIN, bool STAGED, int NBUF = 0>
__device__ void build_vertex_merge(u32 t, u32 v, u32 off, u32 n, const float* w,
                                   Slot* __restrict__ slots, uint8_t* __restrict__ valid, u64* A,
                                   u32* P, u64* s_tmp, unsigned char* win_smem, u32* err,
                                   TilePipe* pipe = nullptr) {
  auto weight = [&](u32 p) { return sane_weight(STAGED ? w[p] : __ldg(w + p)); };
  float wmax = 0.0f;
  for (u32 p = t; p < n; p += NT) wmax = fmaxf(wmax, weight(p));
  wmax = coop_max<NT>(wmax, reinterpret_cast<float*>(s_tmp));
  if (!(wmax > 0.0f)) {
    for (u32 p = t; p < n; p += NT) slots[(u64)off + p] = Slot{-1.0f, p};
    if (t == 0) valid[v] = 0;
    return;
  }
  const int B = bucket_bits(n);
  const u64 C = (u64)1 << B;
  const int sh = weight_shift(wmax, B);
  u64 W = 0;
  {
    u64 acc = 0;
    for (u32 p = t; p < n; p += NT) acc += quantise_bits(weight(p), sh);
    // total only: the exclusive prefix is not needed here
    u64 x = acc;
    coop_scan_u64<NT>(x, W, s_tmp);
  }
  const u64 nC = (u64)n << B;
  const double K = mass_factor(n, B, W);

  // Only the deficit prefix D and the count of larges are scanned; the excess prefix follows from the
  // cumulative mass: sum over k <= p of (M_k - C) = X(p) - D(p), so X(p) = D(p) + g(Q_(p+1)) - (p + 1) * C.
  u64 cQ = 0, cD = 0;  // carries between tiles (the same value in every thread)
  u32 cL = 0;
  constexpr u32 kTile = NT * EPT;
  constexpr bool BULK = NBUF > 0;
  // BULK: element i of a tile sits at buffer[head + i]; the list starts `head` floats after a 16-byte
  // boundary and tiles are whole multiples of 16 bytes, so every tile has the same head.  The copy
  // engine brings the 16-byte groups that lie inside the tile, up to three floats at either end come
  // with plain loads.
  const u32 head = BULK ? (u32)((reinterpret_cast<uintptr_t>(w) & 15u) >> 2) : 0u;
  auto stage_tile = [&](u32 base, u32 b) {
    if constexpr (BULK) {
      const u32 tile_n = min(kTile, n - base);
      const float* src = w + base;
      float* dst = pipe->buf + b * (kTile + 8);
      const u32 skip = head ? 4u : 0u;                 // floats from the aligned start to the first boundary inside
      const u32 body = (head + tile_n) & ~3u;          // ... and to the last boundary inside
      const u32 lead = head ? min(4u - head, tile_n) : 0u;
      if (t < lead) dst[head + t] = __ldg(src + t);
      if (body > skip) {
        if (t == 0) bulk_copy_g2s(dst + skip, src - head + skip, (body - skip) * 4u, pipe->bars + b);
        const u32 tail = head + tile_n - body;         // elements after the last boundary
        if (t < tail) dst[body + t] = __ldg(src + (body - head) + t);
      } else {
        for (u32 i = lead + t; i < tile_n; i += NT) dst[head + i] = __ldg(src + i);
        if (t == 0) mbar_arrive(pipe->bars + b);       // the phase still has to complete
      }
    }
  };
  if constexpr (BULK) stage_tile(0, 0);
  for (u32 base = 0; base < n; base += NT * EPT) {
    // a ragged last tile spreads its elements over all threads (ept each) instead of filling the first ones
    const u32 ept = min((u32)EPT, (n - base + NT - 1) / NT);
    const u32 p0 = base + t * ept;
    const float* tw = nullptr;  // BULK: this tile's weights in shared memory, tw[i] = weight base + i
    if constexpr (BULK) {
      const u32 b = NBUF == 2 ? (base / kTile) & 1u : 0u;
      // two buffers: the other one was last read in the tile before this one, which ended with a barrier
      if (NBUF == 2 && base + kTile < n) stage_tile(base + kTile, b ^ 1u);
      const bool ok = mbar_wait(pipe->bars + b, (pipe->parity >> b) & 1u, 1u << 16);
      // the same outcome in every thread (and the barrier that publishes the plain stores)
      if (!__syncthreads_and(ok ? 1 : 0)) {
        // record it, give the copies in flight one more bounded chance to land so that nothing still
        // writes this CTA's shared memory when it leaves, and stop
        if (t == 0) dev_fail(err, DEV_ERR_WAIT, v, base, 13);
        if (!ok) mbar_wait(pipe->bars + b, (pipe->parity >> b) & 1u, 1u << 16);
        if (NBUF == 2 && base + kTile < n) mbar_wait(pipe->bars + (b ^ 1u), (pipe->parity >> (b ^ 1u)) & 1u, 1u << 16);
        pipe->failed = true;
        return;
      }
      pipe->parity ^= 1u << b;
      tw = pipe->buf + b * (kTile + 8) + head;
    }
    u64 m[EPT];
    u64 Qex = 0;
#pragma unroll
    for (int k = 0; k < EPT; ++k) {
      m[k] = 0;
      if ((u32)k < ept && p0 + k < n)
        m[k] = quantise_bits(BULK ? sane_weight(tw[p0 + k - base]) : weight(p0 + k), sh);
      Qex += m[k];
    }
    u64 tq;
    coop_scan_u64<NT>(Qex, tq, s_tmp);
    // one buffer: every thread has passed the scan's barriers, so nobody reads this tile's weights any
    // more and the next tile can come in under the rest of this one's work
    if (NBUF == 1 && base + kTile < n) stage_tile(base + kTile, 0);
    Qex += cQ;
    cQ += tq;
    const u64 gex = cum_mass(Qex, W, nC, K);
    u64 g_prev = gex, Q = Qex;
    u64 sd = 0;
    u32 sl = 0;
#pragma unroll
    for (int k = 0; k < EPT; ++k) {
      if ((u32)k < ept && p0 + k < n) {
        Q += m[k];
        const u64 g = cum_mass(Q, W, nC, K);
        m[k] = g - g_prev;
        g_prev = g;
        if (m[k] < C) sd += C - m[k];
        else ++sl;
      }
    }
    u64 td;
    u32 tl;
    coop_scan2<NT>(sd, sl, td, tl, s_tmp);
    u64 Dr = sd + cD, gc = gex;
    u32 Lr = sl + cL;
    const u32 L0 = cL;  // larges before this tile
    cD += td;
    cL += tl;
    if constexpr (WIN == 0) {
#pragma unroll
      for (int k = 0; k < EPT; ++k) {
        const u32 p = p0 + k;
        if ((u32)k < ept && p < n) {
          gc += m[k];
          if (m[k] < C) {
            Dr += C - m[k];
            const u32 i = p - Lr;  // smalls before p
            A[i] = Dr;
            P[i] = p;
          } else {
            const u32 j = Lr++;    // larges before p
            A[n - 1 - j] = Dr + gc - ((u64)(p + 1) << B);
            P[n - 1 - j] = p;
          }
        }
      }
    } else {
      // The lists live in global memory.  A thread's eight entries would go out as eight scattered
      // 8-byte stores per warp instruction; instead the tile's entries are laid out in shared memory
      // first (its smalls from the front, its larges from the back, as in the lists themselves) and
      // copied out with consecutive lanes on consecutive addresses.
      static_assert(WIN == 0 || WIN >= NT * EPT, "the window buffer doubles as the tile's staging area");
      u64* tA = reinterpret_cast<u64*>(win_smem);
      u32* tP = reinterpret_cast<u32*>(tA + WIN);
      const u32 tile_n = min((u32)(NT * EPT), n - base);
#pragma unroll
      for (int k = 0; k < EPT; ++k) {
        const u32 p = p0 + k;
        if ((u32)k < ept && p < n) {
          gc += m[k];
          if (m[k] < C) {
            Dr += C - m[k];
            const u32 i = (p - base) - (Lr - L0);  // smalls of this tile before p
            tA[i] = Dr;
            tP[i] = p;
          } else {
            const u32 j = Lr++ - L0;               // larges of this tile before p
            tA[tile_n - 1 - j] = Dr + gc - ((u64)(p + 1) << B);
            tP[tile_n - 1 - j] = p;
          }
        }
      }
      coop_sync<NT>();
      const u32 ts = tile_n - tl;          // smalls in this tile
      const u32 S0 = base - L0;            // smalls before this tile
      for (u32 x = t; x < ts; x += NT) {
        A[S0 + x] = tA[x];
        P[S0 + x] = tP[x];
      }
      for (u32 x = t; x < tl; x += NT) {   // large L0 + x sits at n - 1 - (L0 + x)
        A[n - 1 - (L0 + x)] = tA[tile_n - 1 - x];
        P[n - 1 - (L0 + x)] = tP[tile_n - 1 - x];
      }
      coop_sync<NT>();
    }
  }
  coop_sync<NT>();
  const u32 L = cL, S = n - L;
  if (L == 0) {  // mass conservation guarantees a large
    if (t == 0) dev_fail(err, DEV_ERR_INTERNAL, v, L, 7);
    for (u32 p = t; p < n; p += NT) slots[(u64)off + p] = Slot{1.0f, p};
    if (t == 0) valid[v] = 1;
    return;
  }
  if constexpr (WIN == 0) {
    merge_window<NT>(t, n, S, A, P, 0, kNoNext, C, B, off, slots, v, err);
  } else {
    // Lists live in global scratch: cut the merged order into windows of WIN outputs, stage each
    // window's two list slices in shared memory with coalesced copies and merge it from there.
    u64* sA = reinterpret_cast<u64*>(win_smem);
    u32* sP = reinterpret_cast<u32*>(sA + WIN);
    u32* bnd = sP + WIN;  // smalls before the start of each window of one round (NT + 1 entries)
    const u32 nwin = (n + WIN - 1) / WIN;
    for (u32 w0 = 0; w0 < nwin; w0 += NT - 1) {  // a round of cnt windows needs cnt + 1 boundaries
      const u32 cnt = min((u32)NT - 1, nwin - w0);
      coop_sync<NT>();
      if (t <= cnt) {  // one bisection per window boundary, all in parallel
        const u32 k0 = min((w0 + t) * (u32)WIN, n);
        u32 lo = k0 > L ? k0 - L : 0, hi = min(k0, S);
        while (lo < hi) {
          const u32 mid = (lo + hi) >> 1;
          const u64 a = mid ? A[mid - 1] : 0;
          const u64 b = A[n - 1 - (k0 - 1 - mid)];
          if (a <= b) lo = mid + 1;
          else hi = mid;
        }
        bnd[t] = lo;
      }
      coop_sync<NT>();
      for (u32 wi = 0; wi < cnt; ++wi) {
        const u32 k0 = (w0 + wi) * (u32)WIN, k1 = min(k0 + (u32)WIN, n);
        const u32 i0 = bnd[wi], i1 = bnd[wi + 1];
        const u32 j0 = k0 - i0, j1 = k1 - i1;
        const u32 Sl = i1 - i0, Ll = j1 - j0, nl = Sl + Ll;
        for (u32 x = t; x < Sl; x += NT) {
          sA[x] = A[i0 + x];
          sP[x] = P[i0 + x];
        }
        for (u32 x = t; x < Ll; x += NT) {  // larges j0..j1-1 sit at global n-j1 .. n-j0-1
          sA[Sl + x] = A[n - j1 + x];
          sP[Sl + x] = P[n - j1 + x];
        }
        const u64 dsx_in = i0 ? A[i0 - 1] : 0;
        const u32 next_pos = j1 < L ? P[n - 1 - j1] : kNoNext;
        coop_sync<NT>();
        merge_window<NT>(t, nl, Sl, sA, sP, dsx_in, next_pos, C, B, off, slots, v, err);
        coop_sync<NT>();
      }
    }
  }
  if (t == 0) valid[v] = 1;
}

// ------------------------------------------------------------------ packed lists (n <= 4096) --
// Lists of at most 4096 elements get a leaner form of the same construction.
//   * One list entry is one 64-bit word: (prefix key << 12) | position.  With n <= 4096 the bucket
//     has 40 bits, every prefix stays below 2^52 and a position needs 12 bits, so the merge reads
//     and compares single words (8 instead of 12 bytes of shared memory per edge).
//   * Only the deficit prefix D is scanned, with the number of smalls riding in bits 52..63 of the
//     same word (there is always at least one large, so the count is at most 4095).  The excess prefix
//     follows from the cumulative mass: sum over k <= p of (M_k - C) = X(p) - D(p), hence
//     X(p) = D(p) + g(Q_(p+1)) - (p + 1) * C, with g(Q_(p+1)) already at hand.
//   * Each thread owns EPT consecutive elements of a tile, so the prefix sums are short serial
//     loops plus one cross-thread scan per tile; when the whole list fits one tile (SINGLE) the
//     weights are loaded and quantised once and stay in registers, and the scan of the quantised
//     weights yields their total as well.
//   * The merge keeps the heads of both lists in registers: one shared-memory load per output.
constexpr int kPosBits = 12;
constexpr u64 kPosMask = (1ull << kPosBits) - 1;
constexpr int kCntShift = 52;
constexpr u64 kKeyMask = (1ull << kCntShift) - 1;
constexpr u64 kListEnd = ~0ull;  // stands for "no entry left": its key exceeds every real key
constexpr u32 kPackedMax = 1u << kPosBits;

// Cooperation inside a group of G lanes of one warp (G = 1, 2, 4 ... 32).  Groups of a warp work on
// different vertices and may diverge, so every shuffle names only the lanes of its own group.
template <int G>
struct GroupCoop {
  static constexpr int NT = G;
  u32 mask, t;
  __device__ __forceinline__ GroupCoop() {
    const u32 lane = threadIdx.x & 31;
    t = lane & (G - 1);
    mask = G == 32 ? 0xFFFFFFFFu : (((1u << G) - 1u) << (lane & ~(u32)(G - 1)));
  }
  __device__ __forceinline__ void sync() const { __syncwarp(mask); }
  __device__ __forceinline__ float max(float v) const {
#pragma unroll
    for (int o = G / 2; o; o >>= 1) v = fmaxf(v, __shfl_xor_sync(mask, v, o, G));
    return v;
  }
  __device__ __forceinline__ u64 sum(u64 x) const {
#pragma unroll
    for (int o = G / 2; o; o >>= 1) x += __shfl_xor_sync(mask, x, o, G);
    return x;
  }
  // v becomes the exclusive prefix over the group, total the group's sum
  __device__ __forceinline__ void scan(u64& v, u64& total) const {
    u64 inc = v;
#pragma unroll
    for (int o = 1; o < G; o <<= 1) {
      const u64 x = __shfl_up_sync(mask, inc, o, G);
      if (t >= (u32)o) inc += x;
    }
    total = __shfl_sync(mask, inc, G - 1, G);
    v = inc - v;
  }
};

// Cooperation inside a CTA of NTHREADS threads (s_tmp: NTHREADS / 32 + 1 words of shared memory).
template <int NTHREADS>
struct CtaCoop {
  static constexpr int NT = NTHREADS;
  u32 t;
  u64* s_tmp;
  __device__ __forceinline__ explicit CtaCoop(u64* tmp) : t(threadIdx.x), s_tmp(tmp) {}
  __device__ __forceinline__ void sync() const { __syncthreads(); }
  __device__ __forceinline__ float max(float v) const { return coop_max<NTHREADS>(v, reinterpret_cast<float*>(s_tmp)); }
  __device__ __forceinline__ u64 sum(u64 x) const {
    u64 total;
    coop_scan_u64<NTHREADS>(x, total, s_tmp);
    return total;
  }
  __device__ __forceinline__ void scan(u64& v, u64& total) const { coop_scan_u64<NTHREADS>(v, total, s_tmp); }
};

// Merge of the packed lists: S smalls at A[0 .. S) with key = inclusive deficit prefix, L = n - S
// larges from the back (large j at A[n - 1 - j]) with key = inclusive excess prefix.  Thread t emits
// an equal share of the merged order.  Keys are compared and subtracted where they sit, in bits 12
// and up of an entry (a mass times 2^12 rounds to the same float as the mass, the scale being a
// power of two).  A step of the loop has no branch: the entry that leaves, the entry that names the
// alias and the two keys that make up the mass are selected, and one load refills the window of
// three entries (the small at the head, the large at the head, the large behind it).
template <int NT>
__device__ __forceinline__ void merge_packed(u32 t, u32 n, u32 S, const u64* A, u64 C, int B, u32 off,
                                             Slot* __restrict__ slots, u32 v, u32* err) {
  constexpr u64 kKeyBits = ~kPosMask;
  const u32 L = n - S;
  const u32 VT = (n + NT - 1) / NT;
  const u32 k0 = min(t * VT, n), k1 = min(k0 + VT, n);
  if (k0 >= k1) return;
  u32 i;
  {
    u32 lo = k0 > L ? k0 - L : 0, hi = min(k0, S);
    while (lo < hi) {  // small mid precedes large k0-1-mid iff its key (deficit before it) <= that large's key
      const u32 mid = (lo + hi) >> 1;
      const u64 a = mid ? (A[mid - 1] & kKeyBits) : 0;
      const u64 b = A[n - 1 - (k0 - 1 - mid)] & kKeyBits;
      if (a <= b) lo = mid + 1;
      else hi = mid;
    }
    i = lo;
  }
  // i <= S and j <= L hold from here on, and i + j = k < n: the entry that leaves always exists
  u32 j = k0 - i;
  u64 dsx = i ? (A[i - 1] & kKeyBits) : 0;  // deficit of the smalls before small i
  u64 hs = i < S ? A[i] : kListEnd;
  u64 hl = j < L ? A[n - 1 - j] : kListEnd;
  u64 hl2 = j + 1 < L ? A[n - 2 - j] : kListEnd;
  const u64 Cs = C << kPosBits;
  const int Bs = B + kPosBits;
  Slot* __restrict__ out = slots + off;
  bool bad = false;
  for (u32 k = k0; k < k1; ++k) {
    const u64 ks = hs & kKeyBits, kl = hl & kKeyBits;
    const bool fits = dsx <= kl;           // the large at the head still has room for a small
    const bool take = i < S && fits;       // a small leaves; else a large
    const bool full = !take && fits;       // only once every small is placed: the large owns its bucket
    const u64 e = take ? hs : hl;
    const u64 a = take ? hl : hl2;         // a small's alias is the large at the head, a large's the next one
    const u32 p = (u32)e & (u32)kPosMask;
    // mass conservation puts the last large after every small and leaves no large short of a
    // successor; an entry that is missing all the same is recorded and the slot made self-contained
    const bool none = (u32)(a >> 32) == 0xFFFFFFFFu;  // a key stays below 2^52 - 2^40: only kListEnd has these bits
    bad |= none && !full;
    const bool self = full || none;
    const u64 x = take ? dsx : kl, y = take ? ks : dsx;  // small: C - (ks - dsx); large: kl + C - dsx
    Slot o;
    o.prob = self ? 1.0f : mass_to_prob_fast(Cs + x - y, Bs);
    o.alias = self ? p : ((u32)a & (u32)kPosMask);
    out[p] = o;
    i += take ? 1u : 0u;
    j += take ? 0u : 1u;
    const u32 idx = take ? i : n - 2 - j;
    const bool more = take ? i < S : j + 1 < L;
    const u64 nx = more ? A[idx] : kListEnd;
    dsx = take ? ks : dsx;
    hl = take ? hl : hl2;
    hl2 = take ? hl2 : nx;
    hs = take ? nx : hs;
  }
  if (bad) dev_fail(err, DEV_ERR_INTERNAL, v, k0, 8);
}

// Table of one vertex (degree n <= 4096) by the threads of `co`; A holds n packed list entries.
// SINGLE: n <= NT * EPT.  STAGED: w points at a copy of the weights in shared memory.
template <class Coop, int EPT, bool SINGLE, bool STAGED>
__device__ __forceinline__ void build_vertex_packed(const Coop& co, u32 v, u32 off, u32 n, const float* w,
                                                    Slot* __restrict__ slots, uint8_t* __restrict__ valid,
                                                    u64* A, u32* err) {
  constexpr int NT = Coop::NT;
  const u32 t = co.t;
  auto weight = [&](u32 p) { return sane_weight(STAGED ? w[p] : __ldg(w + p)); };
  float wr[EPT];
  float wmax = 0.0f;
  // SINGLE: the list is one tile, spread evenly over the threads (ceil(n / NT) <= EPT elements each)
  const u32 ept1 = (n + NT - 1) / NT;
  if constexpr (SINGLE) {
    const u32 p1 = t * ept1;
    const u32 cnt1 = p1 < n ? min(ept1, n - p1) : 0u;
#pragma unroll
    for (int k = 0; k < EPT; ++k) {
      wr[k] = (u32)k < cnt1 ? weight(p1 + k) : 0.0f;
      wmax = fmaxf(wmax, wr[k]);
    }
  } else {
    for (u32 p = t; p < n; p += NT) wmax = fmaxf(wmax, weight(p));
  }
  wmax = co.max(wmax);
  if (!(wmax > 0.0f)) {
    for (u32 p = t; p < n; p += NT) slots[(u64)off + p] = Slot{-1.0f, p};
    if (t == 0) valid[v] = 0;
    return;
  }
  const int B = bucket_bits(n);
  const u64 C = (u64)1 << B;
  const int sh = weight_shift(wmax, B);
  u64 m[EPT];
  u64 W = 0, Qex = 0;
  if constexpr (SINGLE) {
#pragma unroll
    for (int k = 0; k < EPT; ++k) {
      m[k] = quantise_bits(wr[k], sh);
      Qex += m[k];
    }
    co.scan(Qex, W);  // one scan gives the prefix of this thread and the total
  } else {
    u64 acc = 0;
    for (u32 p = t; p < n; p += NT) acc += quantise_bits(weight(p), sh);
    W = co.sum(acc);
  }
  const u64 nC = (u64)n << B;
  const double K = mass_factor(n, B, W);
  u64 cQ = 0, cPK = 0;  // carries between tiles (the same value in every thread)
  for (u32 base = 0; base < (SINGLE ? 1u : n); base += NT * EPT) {
    // A ragged last tile spreads its elements over all threads (ept of them each, the same in every
    // thread) instead of filling the first threads with EPT each: a list of 278 weights then costs a
    // warp one tile of 8 elements per lane plus one of 1, not two of 8.
    const u32 ept = SINGLE ? ept1 : min((u32)EPT, (n - base + NT - 1) / NT);
    const u32 p0 = base + t * ept;
    const u32 cnt = p0 < n ? min(ept, n - p0) : 0u;  // elements of this thread in this tile
    if constexpr (!SINGLE) {
      Qex = 0;
#pragma unroll
      for (int k = 0; k < EPT; ++k) {
        m[k] = 0;
        if ((u32)k < cnt) m[k] = quantise_bits(weight(p0 + k), sh);
        Qex += m[k];
      }
      u64 tq;
      co.scan(Qex, tq);
      Qex += cQ;
      cQ += tq;
    }
    const u64 gex = cum_mass(Qex, W, nC, K);  // cumulative mass before this thread's elements
    u64 g_prev = gex, Q = Qex, pk = 0;
#pragma unroll
    for (int k = 0; k < EPT; ++k) {
      if ((u32)k < cnt) {
        Q += m[k];
        const u64 g = cum_mass(Q, W, nC, K);
        m[k] = g - g_prev;
        g_prev = g;
        if (m[k] < C) pk += (C - m[k]) + (1ull << kCntShift);
      }
    }
    u64 tpk;
    co.scan(pk, tpk);
    pk += cPK;
    cPK += tpk;
    u64 Dr = pk & kKeyMask, gc = gex;
    u32 Sr = (u32)(pk >> kCntShift);  // smalls before this thread's elements
#pragma unroll
    for (int k = 0; k < EPT; ++k) {
      const u32 p = p0 + k;
      if ((u32)k < cnt) {
        gc += m[k];
        const bool small = m[k] < C;
        Dr += small ? C - m[k] : 0ull;
        // a small carries the inclusive deficit prefix, a large the inclusive excess prefix
        const u64 key = small ? Dr : Dr + gc - ((u64)(p + 1) << B);
        const u32 at = small ? Sr : n - 1 - (p - Sr);
        Sr += small ? 1u : 0u;
        A[at] = (key << kPosBits) | p;
      }
    }
  }
  co.sync();
  const u32 S = (u32)(cPK >> kCntShift);
  if (S >= n) {  // mass conservation guarantees a large
    if (t == 0) dev_fail(err, DEV_ERR_INTERNAL, v, S, 7);
    for (u32 p = t; p < n; p += NT) slots[(u64)off + p] = Slot{1.0f, p};
    if (t == 0) valid[v] = 1;
    return;
  }
  merge_packed<NT>(t, n, S, A, C, B, off, slots, v, err);
  if (t == 0) valid[v] = 1;
}

// Degrees up to 8 * G: one group of G lanes per vertex, 32 / G vertices per warp side by side, the
// whole list in registers.  Every warp owns 256 list words of shared memory, 8 * G per group.
template <int G>
__global__ void __launch_bounds__(256) build_small_kernel(const u32* __restrict__ worklist,
                                                          const u32* __restrict__ cls, int k,
                                                          const u32* __restrict__ xadj,
                                                          const float* __restrict__ wgt,
                                                          Slot* __restrict__ slots,
                                                          uint8_t* __restrict__ valid,
                                                          u32* __restrict__ err) {
  __shared__ u64 s_lists[8][32 * kGroupEpt];
  const u32 count = cls[k], base = cls[2 * K_CLASSES + k];
  const u32 lane = threadIdx.x & 31;
  constexpr u32 GPW = 32 / G;  // groups per warp
  const u32 warp_id = (blockIdx.x * blockDim.x + threadIdx.x) >> 5;
  const u32 nwarps = (gridDim.x * blockDim.x) >> 5;
  u64* A = s_lists[threadIdx.x >> 5] + (lane / G) * (G * kGroupEpt);
  const GroupCoop<G> co;
  for (u64 it0 = (u64)warp_id * GPW; it0 < count; it0 += (u64)nwarps * GPW) {
    const u64 it = it0 + lane / G;
    if (it < count) {
      const u32 v = worklist[base + it];
      const u32 off = xadj[v], n = xadj[v + 1] - off;
      if (n > G * kGroupEpt || n == 0) {  // classification and kernel disagree: record and skip
        if (co.t == 0) dev_fail(err, DEV_ERR_INTERNAL, v, n, G);
      } else {
        build_vertex_packed<GroupCoop<G>, (int)kGroupEpt, true, false>(co, v, off, n, wgt + off, slots, valid, A, err);
      }
      co.sync();  // the group's list words are reused by its next vertex
    }
  }
}

// Degrees 257 .. 1024: one warp per vertex (tiles of 256 elements), WPB warps per CTA, vertices
// handed out by an atomic cursor because their cost varies with the degree.
template <int CAP, int WPB>
__global__ void __launch_bounds__(WPB * 32) build_warp_packed_kernel(const u32* __restrict__ worklist,
                                                                     u32* __restrict__ cls, int k,
                                                                     const u32* __restrict__ xadj,
                                                                     const float* __restrict__ wgt,
                                                                     Slot* __restrict__ slots,
                                                                     uint8_t* __restrict__ valid,
                                                                     u32* __restrict__ err) {
  extern __shared__ __align__(16) unsigned char smem[];
  const u32 count = cls[k], base = cls[2 * K_CLASSES + k];
  const u32 lane = threadIdx.x & 31, wib = threadIdx.x >> 5;
  u64* A = reinterpret_cast<u64*>(smem) + (size_t)wib * CAP;
  u32* cursor = cls + 3 * K_CLASSES + k;
  const GroupCoop<32> co;
  for (;;) {
    u32 it = 0;
    if (lane == 0) it = atomicAdd(cursor, 1u);
    it = __shfl_sync(0xFFFFFFFFu, it, 0);
    if (it >= count) break;
    const u32 v = worklist[base + it];
    const u32 off = xadj[v], n = xadj[v + 1] - off;
    if (n > CAP || n == 0) {
      if (lane == 0) dev_fail(err, DEV_ERR_CAPACITY, v, n, CAP);
      continue;
    }
    build_vertex_packed<GroupCoop<32>, 8, false, false>(co, v, off, n, wgt + off, slots, valid, A, err);
    __syncwarp();
  }
}

// Degrees 1025 .. 4096 when the weight array cannot be bulk-copied (not 16-byte aligned): one CTA
// of NT threads per vertex, weights read from global memory.
template <int NT>
__global__ void __launch_bounds__(NT) build_cta_packed_kernel(const u32* __restrict__ worklist,
                                                              u32* __restrict__ cls, int k,
                                                              const u32* __restrict__ xadj,
                                                              const float* __restrict__ wgt,
                                                              Slot* __restrict__ slots,
                                                              uint8_t* __restrict__ valid,
                                                              u32* __restrict__ err) {
  extern __shared__ __align__(16) unsigned char smem[];
  __shared__ u64 s_tmp[NT / 32 + 1];
  __shared__ u32 s_it;
  u64* A = reinterpret_cast<u64*>(smem);
  const u32 count = cls[k], base = cls[2 * K_CLASSES + k];
  const CtaCoop<NT> co(s_tmp);
  for (;;) {
    if (threadIdx.x == 0) s_it = atomicAdd(cls + 3 * K_CLASSES + k, 1u);
    __syncthreads();
    const u32 it = s_it;
    __syncthreads();
    if (it >= count) break;
    const u32 v = worklist[base + it];
    const u32 off = xadj[v], n = xadj[v + 1] - off;
    if (n > kPackedMax || n == 0) {
      if (threadIdx.x == 0) dev_fail(err, DEV_ERR_CAPACITY, v, n, kPackedMax);
      continue;
    }
    build_vertex_packed<CtaCoop<NT>, 8, false, false>(co, v, off, n, wgt + off, slots, valid, A, err);
    __syncthreads();
  }
}

// Dynamic shared memory of the scratch class: the merge windows (WIN keys and positions, NT + 1
// window boundaries), rounded up to 16 bytes, then two weight tiles of NT * 8 + 8 floats.
__host__ __device__ constexpr int win_smem_bytes(int nt, int win) { return (win * 12 + (nt + 1) * 4 + 15) & ~15; }
__host__ __device__ constexpr int tile_pipe_bytes(int nt) { return 2 * (nt * 8 + 8) * 4; }

// One CTA of NT threads per vertex of degree <= cap.  WIN == 0: lists in dynamic shared memory.
// WIN > 0: lists in this CTA's slab of global scratch (cap entries of 12 bytes), merged through
// windows of WIN outputs staged in dynamic shared memory.
template <int NT, int WIN>
__global__ void __launch_bounds__(NT) build_cta_merge_kernel(const u32* __restrict__ worklist,
                                                             u32* __restrict__ cls, int k,
                                                             const u32* __restrict__ xadj,
                                                             const float* __restrict__ wgt,
                                                             Slot* __restrict__ slots,
                                                             uint8_t* __restrict__ valid,
                                                             unsigned char* __restrict__ scratch,
                                                             u64 cap, u32* __restrict__ err) {
  extern __shared__ __align__(16) unsigned char smem[];
  __shared__ u64 s_tmp[2 * (NT / 32 + 1)];
  __shared__ __align__(8) u64 s_bars[2];
  unsigned char* store = WIN ? scratch + (u64)blockIdx.x * cap * 12ull : smem;
  u64* A = reinterpret_cast<u64*>(store);
  u32* P = reinterpret_cast<u32*>(A + cap);
  const u32 count = cls[k], base = cls[2 * K_CLASSES + k];
  __shared__ u32 s_it;
  // Weight tiles brought in by the bulk-copy engine: two buffers behind the merge windows (WIN > 0), one
  // buffer behind the lists of the shared-memory classes (two 512-thread CTAs with 96 KB of lists and a
  // 16 KB tile each still share an SM)
  constexpr int NBUF = WIN > 0 ? 2 : 1;
  TilePipe pipe{reinterpret_cast<float*>(WIN ? smem + win_smem_bytes(NT, WIN) : smem + cap * 12ull), s_bars, 0u, false};
  if (NBUF && threadIdx.x == 0) {
    mbar_init(&s_bars[0], 1);
    mbar_init(&s_bars[1], 1);
  }
  __syncthreads();
  for (;;) {  // next vertex from the class's atomic cursor (degrees, hence costs, vary widely)
    if (threadIdx.x == 0) s_it = atomicAdd(cls + 3 * K_CLASSES + k, 1u);
    __syncthreads();
    const u32 it = s_it;
    __syncthreads();
    if (it >= count) break;
    const u32 v = worklist[base + it];
    const u32 off = xadj[v], n = xadj[v + 1] - off;
    if (n > cap) {
      if (threadIdx.x == 0) dev_fail(err, DEV_ERR_CAPACITY, v, n, (u32)cap);
      continue;
    }
    build_vertex_merge<NT, 8, WIN, false, NBUF>(threadIdx.x, v, off, n, wgt + off, slots, valid, A, P, s_tmp,
                                                      smem, err, &pipe);
    if (pipe.failed) break;  // the same in every thread
    __syncthreads();
  }
}

// The 1025..CAP class with the weight list staged in shared memory by the bulk-copy engine: one
// cp.async.bulk per vertex brings the 16-byte-aligned middle of the list (the up to 3 floats
// before the first and after the last boundary come with plain loads), the three passes over the
// weights then read shared memory.  The packed lists (8 B/edge) precede the weights in dynamic
// shared memory.
template <int NT, int CAP>
__global__ void __launch_bounds__(NT) build_cta_staged_kernel(const u32* __restrict__ worklist,
                                                              u32* __restrict__ cls, int k,
                                                              const u32* __restrict__ xadj,
                                                              const float* __restrict__ wgt,
                                                              Slot* __restrict__ slots,
                                                              uint8_t* __restrict__ valid,
                                                              u32* __restrict__ err) {
  extern __shared__ __align__(16) unsigned char smem[];
  __shared__ u64 s_tmp[NT / 32 + 1];
  __shared__ __align__(8) u64 s_bar;
  __shared__ u32 s_it;
  u64* A = reinterpret_cast<u64*>(smem);
  float* sW = reinterpret_cast<float*>(A + CAP);  // CAP + 8 floats, 16-byte aligned
  const CtaCoop<NT> co(s_tmp);
  const u32 count = cls[k], base = cls[2 * K_CLASSES + k];
  if (threadIdx.x == 0) mbar_init(&s_bar, 1);
  __syncthreads();
  u32 parity = 0;
  for (;;) {
    if (threadIdx.x == 0) s_it = atomicAdd(cls + 3 * K_CLASSES + k, 1u);
    __syncthreads();
    const u32 it = s_it;
    __syncthreads();
    if (it >= count) break;
    const u32 v = worklist[base + it];
    const u32 off = xadj[v], n = xadj[v + 1] - off;
    if (n > (u32)CAP || n == 0) {
      if (threadIdx.x == 0) dev_fail(err, DEV_ERR_CAPACITY, v, n, CAP);
      continue;
    }
    const float* w = wgt + off;
    const u32 head = (u32)((reinterpret_cast<uintptr_t>(w) & 15u) >> 2);            // floats before w in its 16-byte group
    const float* first = w - head;                                                 // aligned start
    const u32 body = ((head + n) & ~3u);                                           // floats up to the last boundary
    const u32 lead = head ? 4 - head : 0;                                          // list elements before the first boundary
    // elements [lead_start .. ) layout in sW: element i of the list lives at sW[head + i]
    bool mine_ok = true;
    const u32 skip = head ? 4u : 0u;  // floats from `first` to the first boundary inside the list
    const bool bulk = body > skip;
    if (bulk) {
      // whole 16-byte groups that lie inside the list: [first + skip, first + body)
      if (threadIdx.x == 0) bulk_copy_g2s(sW + skip, first + skip, (body - skip) * 4u, &s_bar);
      // ragged ends by plain loads
      if (threadIdx.x < lead) sW[head + threadIdx.x] = __ldg(w + threadIdx.x);
      const u32 tail = head + n - body;  // elements after the last boundary
      if (threadIdx.x < tail) sW[body + threadIdx.x] = __ldg(first + body + threadIdx.x);
      mine_ok = mbar_wait(&s_bar, parity, 1u << 16);
    } else {
      for (u32 i = threadIdx.x; i < n; i += NT) sW[head + i] = __ldg(w + i);
    }
    // the same outcome in every thread (and the barrier that publishes the plain stores)
    if (!__syncthreads_and(mine_ok ? 1 : 0)) {
      // the copy did not report completion in time: record it, give it one more bounded chance to
      // land so that nothing still writes this CTA's shared memory when it leaves, and stop
      if (threadIdx.x == 0) dev_fail(err, DEV_ERR_WAIT, v, n, 12);
      if (!mine_ok) mbar_wait(&s_bar, parity, 1u << 16);
      break;
    }
    if (bulk) parity ^= 1u;
    build_vertex_packed<CtaCoop<NT>, 8, false, true>(co, v, off, n, sW + head, slots, valid, A, err);
    __syncthreads();
  }
}

// ------------------------------------------------------------------ one CTA per vertex -----
template <int T>
__device__ __forceinline__ u64 block_sum(u64 x, u64* s_red) {
#pragma unroll
  for (int o = 16; o; o >>= 1) x += __shfl_xor_sync(0xFFFFFFFFu, x, o);
  __syncthreads();  // s_red may still be read from the previous reduction
  if ((threadIdx.x & 31) == 0) s_red[threadIdx.x >> 5] = x;
  __syncthreads();
  u64 t = 0;
#pragma unroll
  for (int w = 0; w < T / 32; ++w) t += s_red[w];
  return t;
}
template <int T>
__device__ __forceinline__ float block_max(float x, float* s_red) {
#pragma unroll
  for (int o = 16; o; o >>= 1) x = fmaxf(x, __shfl_xor_sync(0xFFFFFFFFu, x, o));
  __syncthreads();
  if ((threadIdx.x & 31) == 0) s_red[threadIdx.x >> 5] = x;
  __syncthreads();
  float t = 0.0f;
#pragma unroll
  for (int w = 0; w < T / 32; ++w) t = fmaxf(t, s_red[w]);
  return t;
}

// First index in [0, n) with a[i] >= t (a non-decreasing); n when there is none.
template <typename V>
__device__ __forceinline__ u32 lower_bound_dev(const V* a, u32 n, V t) {
  u32 lo = 0, hi = n;
  while (lo < hi) {
    const u32 mid = lo + ((hi - lo) >> 1);
    if (a[mid] < t) lo = mid + 1;
    else hi = mid;
  }
  return lo;
}

// Builds the table of one vertex with T threads.  D, X (u64) and LR (u32) hold n entries each,
// in shared memory or in a global slab.
template <int T>
__device__ void build_vertex_cta(u32 v, u32 off, u32 n, const float* __restrict__ wgt,
                                 Slot* __restrict__ slots, uint8_t* __restrict__ valid, u64* D,
                                 u64* X, u32* LR, u64* s_red, u32* err) {
  const u32 tid = threadIdx.x;
  const float* w = wgt + off;
  float wmax = 0.0f;
  for (u32 i = tid; i < n; i += T) wmax = fmaxf(wmax, sane_weight(__ldg(w + i)));
  wmax = block_max<T>(wmax, reinterpret_cast<float*>(s_red));
  if (!(wmax > 0.0f)) {
    for (u32 i = tid; i < n; i += T) slots[(u64)off + i] = Slot{-1.0f, i};
    if (tid == 0) valid[v] = 0;
    return;
  }
  const int B = bucket_bits(n);
  const u64 C = (u64)1 << B;
  const double scale = weight_scale(wmax, B);
  u64 acc = 0;
  for (u32 i = tid; i < n; i += T) acc += quantise(sane_weight(__ldg(w + i)), scale);
  const u64 W = block_sum<T>(acc, s_red);
  const double K = mass_factor(n, B, W);
  const u64 nC = (u64)n << B;

  // tile-wise inclusive scans: first the quantised weights (-> masses), then deficit, excess and
  // large count
  __shared__ u64 s_wq[T / 32], s_wd[T / 32], s_wx[T / 32];
  __shared__ u32 s_wl[T / 32];
  __shared__ u64 s_cq, s_cd, s_cx;
  __shared__ u32 s_cl;
  if (tid == 0) {
    s_cq = 0;
    s_cd = 0;
    s_cx = 0;
    s_cl = 0;
  }
  __syncthreads();
  const u32 lane = tid & 31, warp = tid >> 5;
  for (u32 t0 = 0; t0 < n; t0 += T) {
    const u32 i = t0 + tid;
    const u64 q = i < n ? quantise(sane_weight(__ldg(w + i)), scale) : 0;
    u64 Qi = q;
#pragma unroll
    for (int o = 1; o < 32; o <<= 1) {
      const u64 tq = __shfl_up_sync(0xFFFFFFFFu, Qi, o);
      if (lane >= (u32)o) Qi += tq;
    }
    if (lane == 31) s_wq[warp] = Qi;
    __syncthreads();
    u64 bq = s_cq;
    for (u32 ww = 0; ww < warp; ++ww) bq += s_wq[ww];
    Qi += bq;
    u64 d = 0, x = 0;
    u32 l = 0;
    if (i < n) {
      const u64 m = cum_mass(Qi, W, nC, K) - cum_mass(Qi - q, W, nC, K);
      if (m < C) d = C - m;
      else {
        x = m - C;
        l = 1;
      }
    }
#pragma unroll
    for (int o = 1; o < 32; o <<= 1) {
      const u64 td = __shfl_up_sync(0xFFFFFFFFu, d, o);
      const u64 tx = __shfl_up_sync(0xFFFFFFFFu, x, o);
      const u32 tl = __shfl_up_sync(0xFFFFFFFFu, l, o);
      if (lane >= (u32)o) {
        d += td;
        x += tx;
        l += tl;
      }
    }
    if (lane == 31) {
      s_wd[warp] = d;
      s_wx[warp] = x;
      s_wl[warp] = l;
    }
    __syncthreads();
    u64 bd = s_cd, bx = s_cx;
    u32 bl = s_cl;
    for (u32 ww = 0; ww < warp; ++ww) {
      bd += s_wd[ww];
      bx += s_wx[ww];
      bl += s_wl[ww];
    }
    if (i < n) {
      D[i] = d + bd;
      X[i] = x + bx;
      LR[i] = l + bl;
    }
    __syncthreads();
    if (tid == T - 1) {
      s_cq = Qi;
      s_cd = d + bd;
      s_cx = x + bx;
      s_cl = l + bl;
    }
    __syncthreads();
  }

  for (u32 i = tid; i < n; i += T) {
    const u64 Di = D[i], Xi = X[i];
    const u64 Dp = i ? D[i - 1] : 0;
    const u32 Li = LR[i], Lp = i ? LR[i - 1] : 0;
    Slot out;
    if (Li == Lp) {  // small
      const u64 d = Di - Dp;
      u32 p = Dp ? lower_bound_dev<u64>(X, n, Dp) : lower_bound_dev<u32>(LR, n, 1u);
      if (p >= n) {
        dev_fail(err, DEV_ERR_INTERNAL, v, i, 3);
        p = i;
      }
      out.alias = p;
      out.prob = mass_to_prob(C - d, B);
    } else {
      const u32 S = lower_bound_dev<u64>(D, n, Xi + 1);
      if (S >= n) {
        out.prob = 1.0f;
        out.alias = i;
      } else {
        u32 nx = lower_bound_dev<u32>(LR, n, Li + 1);
        if (nx >= n) {
          dev_fail(err, DEV_ERR_INTERNAL, v, i, 4);
          nx = i;
        }
        out.alias = nx;
        out.prob = mass_to_prob(Xi + C - D[S], B);
      }
    }
    slots[(u64)off + i] = out;
  }
  if (tid == 0) valid[v] = 1;
}

// Launch the class builders over work lists laid out as cls describes (counts at [k],
// bases at [2K + k]).
static int launch_builders(skw_ctx* ctx, const u32* worklist, u32* cls) {
  cudaStream_t st = ctx->stream;
  static_assert(kLargeMax <= kPackedMax, "the 1025+ CTA class uses packed list entries");
  constexpr int kCtaSmem = kLargeMax * 8;
  constexpr int kCta2Smem = kHugeSmemMax * 12 + tile_pipe_bytes(1024) / 2;  // lists + one weight tile
  constexpr int kCta2aSmem = kMidSmemMax * 12 + tile_pipe_bytes(512) / 2;  // lists + one weight tile
  constexpr int kCtaStagedSmem = kLargeMax * 8 + (kLargeMax + 8) * 4;
  constexpr int kW1KSmem = 8 * kWarpMax * 8;
  constexpr int kWin = 8192;                        // merged outputs per window of the scratch class
  constexpr int kWinSmem = win_smem_bytes(1024, kWin) + tile_pipe_bytes(1024);
  static bool attr_set[64] = {false};
  if (!attr_set[ctx->device & 63]) {
    SKW_CUDA(ctx, cudaFuncSetAttribute(build_cta_merge_kernel<1024, kWin>, cudaFuncAttributeMaxDynamicSharedMemorySize, kWinSmem));
    SKW_CUDA(ctx, cudaFuncSetAttribute(build_cta_merge_kernel<1024, 0>, cudaFuncAttributeMaxDynamicSharedMemorySize, kCta2Smem));
    SKW_CUDA(ctx, cudaFuncSetAttribute(build_cta_merge_kernel<512, 0>, cudaFuncAttributeMaxDynamicSharedMemorySize, kCta2aSmem));
    SKW_CUDA(ctx, cudaFuncSetAttribute(build_cta_staged_kernel<256, kLargeMax>,
                                       cudaFuncAttributeMaxDynamicSharedMemorySize, kCtaStagedSmem));
    SKW_CUDA(ctx, cudaFuncSetAttribute(build_warp_packed_kernel<kWarpMax, 8>,
                                       cudaFuncAttributeMaxDynamicSharedMemorySize, kW1KSmem));
    attr_set[ctx->device & 63] = true;
  }
  // one slab per CTA of the scratch class, sized by the largest degree; fewer CTAs when a giant hub
  // would make the slabs exceed 4 GB in total.  (Two 512-thread CTAs per SM instead of one of 1024 were
  // measured: 4.61 against 4.70 ms for this class at scale 26, where thousands of such vertices keep
  // every SM busy either way, but 0.23 ms instead of about 0.15 ms for the largest vertex of an online
  // frontier, which a hop has to wait for; so one vertex gets the 1024 threads.)
  const uint64_t slab_elems = ctx->max_degree > kHugeSmemMax ? (((uint64_t)ctx->max_degree + 1) & ~1ull) : 0;
  int gmem_ctas = ctx->sm_count;
  if (slab_elems) {
    const uint64_t fit = (4ull << 30) / (slab_elems * 12ull);
    if (fit < (uint64_t)gmem_ctas) gmem_ctas = (int)(fit < 8 ? 8 : fit);
  }
  if (slab_elems) {
    int rc = ensure_bytes(ctx, &ctx->cta_scratch, &ctx->cta_scratch_bytes, slab_elems * 12ull * gmem_ctas);
    if (rc != SKW_OK) return rc;
  }
  // The classes are independent and each kernel drains its own work list through an atomic cursor,
  // so they run side by side: the large classes (few, long-running CTAs, whose last vertices would
  // otherwise leave most SMs idle) start first on streams of their own, the small classes fill in
  // on the caller's stream.
  const bool fork = ctx->max_degree > kWarpSmallMax;
  cudaStream_t s_w1k = st, s_c = st, s_c2 = st, s_c2a = st, s_h = st;
  if (fork) {
    SKW_CUDA(ctx, cudaEventRecord(ctx->bfork, st));
    for (int i = 0; i < skw_ctx::kBuilderStreams; ++i) SKW_CUDA(ctx, cudaStreamWaitEvent(ctx->bstream[i], ctx->bfork, 0));
    s_h = ctx->bstream[0];
    s_c2 = ctx->bstream[1];
    s_c = ctx->bstream[2];
    s_w1k = ctx->bstream[3];
    s_c2a = ctx->bstream[3];  // behind the 257-1024 class on its stream
  }
  if (slab_elems) {
    build_cta_merge_kernel<1024, kWin><<<gmem_ctas, 1024, kWinSmem, s_h>>>(
        worklist, cls, K_H, ctx->xadj, ctx->adjwgt, ctx->slots, ctx->valid,
        static_cast<unsigned char*>(ctx->cta_scratch), slab_elems, ctx->d_err);
    SKW_LAUNCHED(ctx);
  }
  if (ctx->max_degree > kMidSmemMax) {
    build_cta_merge_kernel<1024, 0><<<ctx->sm_count, 1024, kCta2Smem, s_c2>>>(
        worklist, cls, K_C2, ctx->xadj, ctx->adjwgt, ctx->slots, ctx->valid, nullptr, kHugeSmemMax, ctx->d_err);
    SKW_LAUNCHED(ctx);
  }
  if (ctx->max_degree > kWarpMax) {
    if ((reinterpret_cast<uintptr_t>(ctx->adjwgt) & 15u) == 0) {
      build_cta_staged_kernel<256, kLargeMax><<<ctx->sm_count * 4, 256, kCtaStagedSmem, s_c>>>(
          worklist, cls, K_C, ctx->xadj, ctx->adjwgt, ctx->slots, ctx->valid, ctx->d_err);
    } else {  // a borrowed weight array that is not 16-byte aligned cannot be bulk-copied
      build_cta_packed_kernel<256><<<ctx->sm_count * 6, 256, kCtaSmem, s_c>>>(
          worklist, cls, K_C, ctx->xadj, ctx->adjwgt, ctx->slots, ctx->valid, ctx->d_err);
    }
    SKW_LAUNCHED(ctx);
  }
  if (ctx->max_degree > kWarpSmallMax) {
    build_warp_packed_kernel<kWarpMax, 8><<<ctx->sm_count * 3, 256, kW1KSmem, s_w1k>>>(
        worklist, cls, K_W1K, ctx->xadj, ctx->adjwgt, ctx->slots, ctx->valid, ctx->d_err);
    SKW_LAUNCHED(ctx);
  }
  if (ctx->max_degree > kLargeMax) {
    build_cta_merge_kernel<512, 0><<<ctx->sm_count * 2, 512, kCta2aSmem, s_c2a>>>(
        worklist, cls, K_C2A, ctx->xadj, ctx->adjwgt, ctx->slots, ctx->valid, nullptr, kMidSmemMax, ctx->d_err);
    SKW_LAUNCHED(ctx);
  }
  const int ggrid = ctx->sm_count * 8;
#define GROUP(GSZ, KCLS)                                                                          \
  if (ctx->max_degree > (GSZ) * kGroupEpt / 2 || (GSZ) == 1) {                                    \
    build_small_kernel<GSZ><<<ggrid, 256, 0, st>>>(worklist, cls, KCLS, ctx->xadj, ctx->adjwgt,   \
                                                   ctx->slots, ctx->valid, ctx->d_err);           \
    SKW_LAUNCHED(ctx);                                                                            \
  }
  GROUP(32, K_G32)
  GROUP(16, K_G16)
  GROUP(8, K_G8)
  GROUP(4, K_G4)
  GROUP(2, K_G2)
  GROUP(1, K_G1)
#undef GROUP
  if (fork) {
    for (int i = 0; i < skw_ctx::kBuilderStreams; ++i) {
      SKW_CUDA(ctx, cudaEventRecord(ctx->bjoin[i], ctx->bstream[i]));
      SKW_CUDA(ctx, cudaStreamWaitEvent(st, ctx->bjoin[i], 0));
    }
  }
  return SKW_OK;
}

// ------------------------------------------------------------------ online frontier --------
// Collect the distinct vertices the live units stand on and bin them by degree class.  Unit u
// reads verts[(u / width) * cells + offs + u % width]; alive (optional) holds kAliveMark for
// units still running.  A vertex is claimed by the first unit that stamps it in the current collection.
constexpr u32 kAliveMark = 0xFFFFFFFFu;

__global__ void frontier_reset_kernel(u32* __restrict__ cls, u32 cap) {
  if (threadIdx.x < K_CLASSES) {
    cls[threadIdx.x] = 0;
    cls[K_CLASSES + threadIdx.x] = 0;
    cls[2 * K_CLASSES + threadIdx.x] = threadIdx.x * cap;
    cls[3 * K_CLASSES + threadIdx.x] = 0;
  }
}

__global__ void __launch_bounds__(256) frontier_collect_kernel(
    const u32* __restrict__ verts, u64 units, u32 width, u32 cells, u32 offs,
    const u32* __restrict__ alive, const u32* __restrict__ xadj, u32 V, u32* __restrict__ stamp,
    u32 round, u32* __restrict__ cls, u32* __restrict__ lists, u32 cap, u32* __restrict__ err) {
  const u32 lane = threadIdx.x & 31;
  const u64 T = (u64)gridDim.x * blockDim.x;
  for (u64 u0 = (u64)blockIdx.x * blockDim.x; u0 < units; u0 += T) {
    const u64 u = u0 + threadIdx.x;
    int c = -1;
    u32 v = 0;
    if (u < units && (!alive || alive[u / width] == kAliveMark)) {
      v = verts[(u / width) * cells + offs + u % width];
      if (v != 0xFFFFFFFFu) {
        if (v >= V) {
          dev_fail(err, DEV_ERR_INDEX, v, (u32)u, 10);
        } else {
          const u32 deg = xadj[v + 1] - xadj[v];
          // a hub stands in thousands of cells of one frontier: look before claiming, so that only the
          // first few of them queue up at its stamp word with an atomic
          if (deg && __ldcg(stamp + v) != round && atomicExch(&stamp[v], round) != round) c = degree_class(deg);
        }
      }
    }
#pragma unroll
    for (int k = 0; k < K_CLASSES; ++k) {
      const u32 m = __ballot_sync(0xFFFFFFFFu, c == k);
      if (!m) continue;
      u32 base = 0;
      if (lane == (u32)(__ffs(m) - 1)) base = atomicAdd(&cls[k], __popc(m));
      base = __shfl_sync(0xFFFFFFFFu, base, __ffs(m) - 1);
      if (c == k) {
        const u32 idx = base + __popc(m & ((1u << lane) - 1u));
        if (idx < cap) lists[(u64)k * cap + idx] = v;
        else dev_fail(err, DEV_ERR_CAPACITY, idx, cap, 11);
      }
    }
  }
}

int frontier_collect(skw_ctx* ctx, const u32* verts, u64 units, u32 width, u32 cells, u32 offs,
                     const u32* alive_lengths, bool new_round) {
  if (units > 0xFFFFFFFFull) return fail(ctx, SKW_ERR_ARG, "frontier of %llu units is too large",
                                         (unsigned long long)units);
  const u32 cap = (u32)(units < ctx->V ? units : ctx->V);
  void* p = ctx->frontier_lists;
  int rc = ensure_bytes(ctx, &p, &ctx->frontier_lists_bytes, sizeof(u32) * (size_t)K_CLASSES * (cap ? cap : 1));
  ctx->frontier_lists = static_cast<u32*>(p);
  if (rc != SKW_OK) return rc;
  if (!ctx->stamp) {
    SKW_CUDA(ctx, cudaMalloc(&ctx->stamp, sizeof(u32) * ((size_t)ctx->V + 1)));
    SKW_CUDA(ctx, cudaMemsetAsync(ctx->stamp, 0, sizeof(u32) * ((size_t)ctx->V + 1), ctx->stream));
    ctx->stamp_round = 0;
  }
  if (!new_round && ctx->stamp_round != 0) {
    // keep the round: vertices claimed earlier in this call are not collected (or built) again
  } else if (++ctx->stamp_round == 0) {  // wrapped: forget every old claim
    SKW_CUDA(ctx, cudaMemsetAsync(ctx->stamp, 0, sizeof(u32) * ((size_t)ctx->V + 1), ctx->stream));
    ctx->stamp_round = 1;
  }
  cudaStream_t st = ctx->stream;
  frontier_reset_kernel<<<1, 32, 0, st>>>(ctx->frontier_cls, cap);
  SKW_LAUNCHED(ctx);
  if (units) {
    // the claim is a chain of dependent accesses (vertex, offsets, stamp): fill every thread slot of the GPU
    const u64 want = (units + 255) / 256;
    const int grid = (int)(want < (u64)ctx->sm_count * 16 ? want : (u64)ctx->sm_count * 16);
    frontier_collect_kernel<<<grid, 256, 0, st>>>(verts, units, width, cells, offs, alive_lengths,
                                                  ctx->xadj, ctx->V, ctx->stamp, ctx->stamp_round,
                                                  ctx->frontier_cls, ctx->frontier_lists, cap, ctx->d_err);
    SKW_LAUNCHED(ctx);
    rc = launch_builders(ctx, ctx->frontier_lists, ctx->frontier_cls);
    if (rc != SKW_OK) return rc;
  }
  return SKW_OK;
}

}  // namespace skw

using namespace skw;

// Self-test of the bounded wait: an mbarrier that nothing ever signals.  The kernel must give up
// after its poll limit, record DEV_ERR_WAIT and return normally.
__global__ void selftest_wait_kernel(u32 limit, u32* err) {
  __shared__ __align__(8) u64 bar;
  if (threadIdx.x == 0) mbar_init(&bar, 1);
  __syncthreads();
  const bool done = mbar_wait(&bar, 0, limit);
  if (!__syncthreads_and(done ? 1 : 0) && threadIdx.x == 0) dev_fail(err, DEV_ERR_WAIT, limit, 0, 99);
}

extern "C" int skw_selftest_bounded_wait(skw_ctx* ctx) {
  if (!ctx) return SKW_ERR_ARG;
  DeviceGuard g(ctx->device);
  int rc = err_reset(ctx);
  if (rc != SKW_OK) return rc;
  selftest_wait_kernel<<<1, 64, 0, ctx->stream>>>(1u << 10, ctx->d_err);
  SKW_LAUNCHED(ctx);
  return err_check(ctx, "skw_selftest_bounded_wait");
}

extern "C" int skw_alias_build_offline(skw_ctx* ctx, uint32_t v_begin, uint32_t v_end, float* ms) {
  if (!ctx) return SKW_ERR_ARG;
  if (!ctx->xadj) return fail(ctx, SKW_ERR_STATE, "skw_alias_build_offline: no graph resident");
  if (!ctx->adjwgt) return fail(ctx, SKW_ERR_STATE, "skw_alias_build_offline: weights were released");
  if (v_begin > v_end || v_end > ctx->V)
    return fail(ctx, SKW_ERR_ARG, "skw_alias_build_offline: vertex range [%u,%u) outside [0,%u]",
                v_begin, v_end, ctx->V);
  DeviceGuard g(ctx->device);
  drop_records(ctx);
  int rc = alloc_table(ctx);
  if (rc != SKW_OK) return rc;
  void* wl = ctx->worklist;
  rc = ensure_bytes(ctx, &wl, &ctx->worklist_cap, sizeof(uint32_t) * ((size_t)ctx->V + 1));
  ctx->worklist = static_cast<uint32_t*>(wl);
  if (rc != SKW_OK) return rc;
  rc = err_reset(ctx);
  if (rc != SKW_OK) return rc;
  cudaStream_t st = ctx->stream;
  SKW_CUDA(ctx, cudaMemsetAsync(ctx->cls_counts, 0, 4 * K_CLASSES * sizeof(uint32_t), st));
  SKW_CUDA(ctx, cudaEventRecord(ctx->ev0, st));
  if (v_end > v_begin) {
    const int cgrid = ctx->sm_count * 8;
    classify_count_kernel<<<cgrid, 256, 0, st>>>(ctx->xadj, v_begin, v_end, ctx->cls_counts, ctx->valid);
    SKW_LAUNCHED(ctx);
    classify_bases_kernel<<<1, 32, 0, st>>>(ctx->cls_counts);
    SKW_LAUNCHED(ctx);
    classify_fill_kernel<<<cgrid, 256, 0, st>>>(ctx->xadj, v_begin, v_end, ctx->cls_counts, ctx->worklist);
    SKW_LAUNCHED(ctx);
    rc = launch_builders(ctx, ctx->worklist, ctx->cls_counts);
    if (rc != SKW_OK) return rc;
  }
  SKW_CUDA(ctx, cudaEventRecord(ctx->ev1, st));
  rc = err_check(ctx, "skw_alias_build_offline");
  if (rc != SKW_OK) return rc;
  if (ms) SKW_CUDA(ctx, cudaEventElapsedTime(ms, ctx->ev0, ctx->ev1));
  ctx->table_ready = true;
  return SKW_OK;
}

// ------------------------------------------------------------------ allocation-free variant --
// skw_alias_build_list_static: the table of ONE weight list, for hosts that must not allocate
// device memory at the time of the call.  Two kinds of caller are meant: a sampler plugged into a
// process whose framework reserved the whole HBM for its own pooling allocator at start-up (a raw
// cudaMalloc from a plug-in then fails, or takes memory behind the pool's back), and a serving
// loop that cannot afford the device-wide synchronisation cudaMalloc / cudaFree imply on its
// request path.  The prefix arrays the CTA builder needs (20 bytes per edge) therefore live in a
// fixed array inside the library image instead of a slab allocated on demand.
namespace skw {

constexpr u32 kStaticMaxDegree = 131072;  // longest weight list the static scratch holds
constexpr size_t kStaticHeader = 256;     // error record, kept apart from the arrays
// 256 B + 131072 * 20 B = 2,621,696 bytes of device memory on every GPU that loads the library,
// held until the process exits.
static __device__ __align__(256) unsigned char g_static_scratch[kStaticHeader + (size_t)kStaticMaxDegree * 20];

// The tile-wise CTA construction (build_vertex_cta) for the single list wgt[0..n), with the prefix arrays
// at `scratch` (the device address of g_static_scratch, looked up by the host).
__global__ void __launch_bounds__(1024) build_list_static_kernel(const float* __restrict__ wgt, u32 n,
                                                                 Slot* __restrict__ slots,
                                                                 uint8_t* __restrict__ valid,
                                                                 unsigned char* __restrict__ scratch) {
  __shared__ u64 s_red[1024 / 32];
  u32* err = reinterpret_cast<u32*>(scratch);
  u64* D = reinterpret_cast<u64*>(scratch + kStaticHeader);
  u64* X = D + kStaticMaxDegree;
  u32* LR = reinterpret_cast<u32*>(X + kStaticMaxDegree);
  build_vertex_cta<1024>(0, 0, n, wgt, slots, valid, D, X, LR, s_red, err);
}

static std::mutex g_static_mu;
static unsigned char* g_static_ptr[64] = {nullptr};  // device address of the array, per device

static int static_fail(char* buf, size_t len, int code, const char* fmt, ...) {
  if (buf && len) {
    va_list ap;
    va_start(ap, fmt);
    vsnprintf(buf, len, fmt, ap);
    va_end(ap);
  }
  return code;
}

}  // namespace skw

extern "C" int skw_alias_build_list_static(const float* d_weights, uint32_t n, void* d_slots,
                                           uint8_t* d_valid, void* cuda_stream, char* errbuf,
                                           size_t errbuf_len) {
  if (errbuf && errbuf_len) errbuf[0] = 0;
  if (!d_weights || !d_slots || !d_valid)
    return static_fail(errbuf, errbuf_len, SKW_ERR_ARG, "skw_alias_build_list_static: null buffer");
  if (n == 0) return static_fail(errbuf, errbuf_len, SKW_ERR_ARG, "skw_alias_build_list_static: empty weight list");
  if (n > kStaticMaxDegree)
    return static_fail(errbuf, errbuf_len, SKW_ERR_ARG,
                       "skw_alias_build_list_static: %u weights exceed the static scratch, which holds %u "
                       "(use skw_alias_build_offline for longer lists)", n, kStaticMaxDegree);
  if ((reinterpret_cast<uintptr_t>(d_slots) & 7u) || (reinterpret_cast<uintptr_t>(d_weights) & 3u))
    return static_fail(errbuf, errbuf_len, SKW_ERR_ARG, "skw_alias_build_list_static: misaligned buffer");
  int dev = -1;
  cudaError_t e = cudaGetDevice(&dev);
  if (e != cudaSuccess)
    return static_fail(errbuf, errbuf_len, SKW_ERR_CUDA, "skw_alias_build_list_static: cudaGetDevice: %s", cudaGetErrorString(e));
  if (dev < 0 || dev >= 64)
    return static_fail(errbuf, errbuf_len, SKW_ERR_ARG, "skw_alias_build_list_static: device %d not supported", dev);
  // a host or peer pointer handed to the kernel would fault: all three buffers must be device memory
  // of the current device
  const void* bufs[3] = {d_weights, d_slots, d_valid};
  const char* names[3] = {"d_weights", "d_slots", "d_valid"};
  for (int i = 0; i < 3; ++i) {
    cudaPointerAttributes at;
    e = cudaPointerGetAttributes(&at, bufs[i]);
    if (e != cudaSuccess || at.type != cudaMemoryTypeDevice || at.device != dev) {
      cudaGetLastError();
      return static_fail(errbuf, errbuf_len, SKW_ERR_ARG,
                         "skw_alias_build_list_static: %s is not device memory of the current device %d", names[i], dev);
    }
  }
  unsigned char* scratch = nullptr;
  {
    // First call on this device: ask the runtime where the array lives on it.  The array's name is
    // only a host-side handle; the kernel must be given this looked-up address.
    std::lock_guard<std::mutex> lk(g_static_mu);
    if (!g_static_ptr[dev]) {
      void* p = nullptr;
      e = cudaGetSymbolAddress(&p, g_static_scratch);
      if (e != cudaSuccess || !p)
        return static_fail(errbuf, errbuf_len, SKW_ERR_CUDA, "skw_alias_build_list_static: cudaGetSymbolAddress: %s",
                           cudaGetErrorString(e));
      g_static_ptr[dev] = static_cast<unsigned char*>(p);
    }
    scratch = g_static_ptr[dev];
  }
  cudaStream_t st = static_cast<cudaStream_t>(cuda_stream);
  // the error record must start at zero; the prefix arrays are fully rewritten before they are read
  e = cudaMemsetAsync(scratch, 0, kStaticHeader, st);
  if (e != cudaSuccess)
    return static_fail(errbuf, errbuf_len, SKW_ERR_CUDA, "skw_alias_build_list_static: cudaMemsetAsync: %s", cudaGetErrorString(e));
  build_list_static_kernel<<<1, 1024, 0, st>>>(d_weights, n, static_cast<Slot*>(d_slots), d_valid, scratch);
  e = cudaGetLastError();
  if (e != cudaSuccess)
    return static_fail(errbuf, errbuf_len, SKW_ERR_CUDA, "skw_alias_build_list_static: launch: %s", cudaGetErrorString(e));
  uint32_t rec[4] = {0, 0, 0, 0};
  e = cudaMemcpyAsync(rec, scratch, sizeof rec, cudaMemcpyDeviceToHost, st);
  if (e == cudaSuccess) e = cudaStreamSynchronize(st);
  if (e != cudaSuccess)
    return static_fail(errbuf, errbuf_len, SKW_ERR_CUDA, "skw_alias_build_list_static: %s", cudaGetErrorString(e));
  if (rec[0] != DEV_OK)
    return static_fail(errbuf, errbuf_len, SKW_ERR_DEVICE,
                       "skw_alias_build_list_static: device error %u, detail %u %u %u", rec[0], rec[1], rec[2], rec[3]);
  return SKW_OK;
}
