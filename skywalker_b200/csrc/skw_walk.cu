// Random-walk step kernels (DeepWalk / PPR / node2vec), offline and online.
//
// Offline: takes over OfflineWalk and sample_kernel_static (src/offline_walk.cu:75-124, 181-230
// of the reference).  One lane carries one walker at a time through all of its steps and picks
// up the next walker of its stride when the current one ends, so lanes stay busy when PPR walks
// stop early; a step is: two offsets, one 8-byte {prob, alias} slot, one neighbour id, one path
// store.  Online: takes over OnlineWalkShMem / OnlineWalkKernel (src/online_walk.cu:82-166,
// 245-327), in one of two ways with identical walks: every walker computes the slot it draws
// straight from the weights (skw_walk_direct.cu), or at every step the tables of the vertices the
// live walkers stand on are built (once per distinct vertex of the frontier, by the degree-bucketed
// builders of skw_alias_build.cu) and every walker draws from the table of its vertex.
//
// Randomness: Philox4x32-10, counter (walker id low, high, step, trial), key seed ^ TAG_WALK;
// word x -> column (multiply-high by the degree), y -> acceptance uniform, z -> PPR stop test,
// w -> node2vec rejection uniform.
#include <algorithm>
#include <cstring>
#include <string>
#include <thread>
#include <vector>

#include <cub/device/device_scan.cuh>
#include <cub/iterator/transform_input_iterator.cuh>

#include "skw_ctx.h"
#include "skw_hostpool.h"
#include "skw_walk_common.cuh"

namespace skw {

int frontier_collect(skw_ctx* ctx, const u32* verts, u64 units, u32 width, u32 cells, u32 offs,
                     const u32* alive_lengths, bool new_round);

// One step of one walker standing on `cur`.  Returns false when the walk ends here.
// r: the random words of (walker, step, trial 0).
template <int APP>
__device__ __forceinline__ bool walk_step(const WalkArgs& a, u64 gw, u32 step, u32 cur, u32 prev,
                                          u32& next, Rand4 r) {
  if (APP == SKW_APP_PPR && u01(r.z) < a.tp) return false;
  if (cur >= a.V) {
    dev_fail(a.err, DEV_ERR_INDEX, cur, step, (u32)gw);
    return false;
  }
  const u32 off = __ldg(a.xadj + cur);
  const u32 deg = __ldg(a.xadj + cur + 1) - off;
  if (deg == 0) return false;
  if (APP == SKW_APP_NODE2VEC && prev != kNoVertex) {
    for (u32 trial = 0;;) {
      const u32 col = __umulhi(r.x, deg);
      u32 cand = col;
      if (!a.unbiased) {
        const Slot s = load_slot(a.slots + (u64)off + col);
        if (s.prob < 0.0f) return false;  // vertex without usable weight
        cand = u01(r.y) < s.prob ? col : s.alias;
        if (cand >= deg) {  // a table that does not belong to this graph
          dev_fail(a.err, DEV_ERR_INDEX, cur, cand, 20);
          return false;
        }
      }
      next = ldg_once(a.adjncy + (u64)off + cand);
      const float f = next == prev ? a.inv_p : (connected(a.xadj, a.adjncy, prev, next) ? 1.0f : a.inv_q);
      if (__fmul_rn(u01(r.w), a.fmax) < f) break;
      if (++trial == kN2vMaxTrials) break;  // keep the last proposal
      r = philox_tagged(a.seed, TAG_WALK, gw, step, trial);
    }
    return true;
  }
  const u32 col = __umulhi(r.x, deg);
  u32 cand = col;
  if (!a.unbiased) {
    const Slot s = load_slot(a.slots + (u64)off + col);
    if (s.prob < 0.0f) return false;
    cand = u01(r.y) < s.prob ? col : s.alias;
    if (cand >= deg) {
      dev_fail(a.err, DEV_ERR_INDEX, cur, cand, 20);
      return false;
    }
  }
  next = ldg_once(a.adjncy + (u64)off + cand);
  return true;
}


// All steps of all walkers in one launch.  Each lane owns walkers tid, tid + T, tid + 2T ...;
// the loop body is one step, so lanes of a warp stay converged although their walkers differ.
template <int APP>
__global__ void __launch_bounds__(256) walk_offline_kernel(const WalkArgs a) {
  const u64 T = (u64)gridDim.x * blockDim.x;
  u64 w = (u64)blockIdx.x * blockDim.x + threadIdx.x;
  u64 edges = 0;
  bool have = w < a.n;
  u32 cur = 0, prev = kNoVertex, step = 0;
  u32* row = nullptr;
  Rand4 r{0, 0, 0, 0};  // random words of the walker's current step
  if (have) {
    cur = __ldg(a.starts + w);
    row = a.paths + w * a.hop_num;
    row[0] = cur;
    if (APP != SKW_APP_PPR) r = philox_tagged(a.seed, TAG_WALK, a.walker_base + w * a.walker_stride, 0, 0);
  }
  while (have) {
    u32 next = 0;
    const u64 gw = a.walker_base + w * a.walker_stride;
    // The next step's words depend on nothing the step loads: computed here, they overlap its chain
    // of dependent loads (40,000 x 80 DeepWalk on the slot table: 153 -> 145 us).  Not for PPR, whose
    // walks mostly end after a step or two: there the words computed ahead are mostly thrown away
    // (8 M walkers: 1.89 -> 1.96 ms), so each step computes its own.
    Rand4 rn{0, 0, 0, 0};
    bool go;
    if (APP == SKW_APP_PPR) {
      go = step + 1 < a.hop_num &&
           walk_step<APP>(a, gw, step, cur, prev, next, philox_tagged(a.seed, TAG_WALK, gw, step, 0));
    } else {
      rn = philox_tagged(a.seed, TAG_WALK, gw, step + 1, 0);
      go = step + 1 < a.hop_num && walk_step<APP>(a, gw, step, cur, prev, next, r);
    }
    if (go) {
      ++step;
      row[step] = next;
      prev = cur;
      cur = next;
      if (APP != SKW_APP_PPR) r = rn;
    } else {
      a.lengths[w] = step;
      edges += step;
      w += T;
      have = w < a.n;
      if (have) {
        cur = __ldg(a.starts + w);
        row = a.paths + w * a.hop_num;
        row[0] = cur;
        prev = kNoVertex;
        step = 0;
        if (APP != SKW_APP_PPR) r = philox_tagged(a.seed, TAG_WALK, a.walker_base + w * a.walker_stride, 0, 0);
      }
    }
  }
  add_edges(a.sum, edges);
}

// Online mode: start of a run (row[0] = start, length = "alive").
__global__ void __launch_bounds__(256) walk_online_init_kernel(const WalkArgs a) {
  for (u64 w = (u64)blockIdx.x * blockDim.x + threadIdx.x; w < a.n; w += (u64)gridDim.x * blockDim.x) {
    a.paths[w * a.hop_num] = __ldg(a.starts + w);
    a.lengths[w] = a.hop_num > 1 ? kAlive : 0u;
  }
}

// Online mode: one step of every live walker, after the tables of the frontier were built.
template <int APP>
__global__ void __launch_bounds__(256) walk_online_step_kernel(const WalkArgs a, u32 step) {
  u64 edges = 0;
  for (u64 w = (u64)blockIdx.x * blockDim.x + threadIdx.x; w < a.n; w += (u64)gridDim.x * blockDim.x) {
    if (a.lengths[w] != kAlive) continue;
    u32* row = a.paths + w * a.hop_num;
    const u32 cur = row[step];
    const u32 prev = (APP == SKW_APP_NODE2VEC && step) ? row[step - 1] : kNoVertex;
    u32 next = 0;
    const u64 gw = a.walker_base + w * a.walker_stride;
    if (walk_step<APP>(a, gw, step, cur, prev, next, philox_tagged(a.seed, TAG_WALK, gw, step, 0))) {
      row[step + 1] = next;
      if (step + 2 == a.hop_num) {
        a.lengths[w] = step + 1;
        edges += step + 1;
      }
    } else {
      a.lengths[w] = step;
      edges += step;
    }
  }
  add_edges(a.sum, edges);
}

// ------------------------------------------------------------------ fused walk records -----
// B200 has room for a wider table: one 32-byte record per edge slot that already holds both
// outcomes of the draw together with what the NEXT step needs (offset and degree of the vertex
// reached), so a step is ONE random 32-byte access (one 256-bit load) instead of three dependent
// ones (offsets -> slot -> neighbour id).  Random DRAM accesses per step, not bytes, bound the
// walk on this memory system, so this is worth 4x the table size.  The records are derived from
// the alias table and the CSR and give bit-identical walks.
//   w0 prob | w1 neighbour if kept | w2 its first-edge offset | w3 its usable degree
//           | w4 neighbour via alias | w5 its offset          | w6 its usable degree | w7 alias
// "usable degree" is 0 for a vertex without out-edges or without usable weight: the walk ends there.
struct __align__(32) WalkRecord {
  u32 w[8];
};

// One 256-bit load.  By default an L1 miss pulls the whole 128-byte line (4 sectors) from DRAM; a
// record is one sector and is used once, so ask for the smallest L2 fetch (64 bytes) and keep it
// out of L1.  Measured on B200: same access rate, half the DRAM traffic.
__device__ __forceinline__ void load_record(const WalkRecord* p, u32 (&w)[8]) {
  asm volatile("ld.global.nc.L1::no_allocate.L2::64B.v8.u32 {%0,%1,%2,%3,%4,%5,%6,%7}, [%8];"
               : "=r"(w[0]), "=r"(w[1]), "=r"(w[2]), "=r"(w[3]), "=r"(w[4]), "=r"(w[5]), "=r"(w[6]), "=r"(w[7])
               : "l"(p));
}

// vinfo[v] = {first-edge offset, usable degree}; vbits = one bit per vertex, set when the usable
// degree is not zero.  The bitmap is V/8 bytes and stays in L2, so a walker that starts on a dead
// end (most uniformly random starts of a directed R-MAT graph) never touches DRAM for it.
__global__ void __launch_bounds__(256) vertex_info_kernel(const u32* __restrict__ xadj,
                                                          const Slot* __restrict__ slots, u32 V,
                                                          uint2* __restrict__ vinfo, u32* __restrict__ vbits,
                                                          u32* __restrict__ unusable) {
  const u64 T = (u64)gridDim.x * blockDim.x;
  const u64 rounds = ((u64)V + T - 1) / T;
  for (u64 it = 0; it < rounds; ++it) {  // whole warps stay in the loop: the ballot needs them
    const u64 v = it * T + (u64)blockIdx.x * blockDim.x + threadIdx.x;
    u32 eff = 0;
    if (v < V) {
      const u32 off = xadj[v], deg = xadj[v + 1] - off;
      eff = deg;
      if (deg && load_slot(slots + off).prob < 0.0f) {
        eff = 0;
        atomicAdd(unusable, 1u);  // has out-edges but no table (all weights unusable, or not built yet): rare
      }
      vinfo[v] = make_uint2(off, eff);
    }
    const u32 word = __ballot_sync(0xFFFFFFFFu, eff != 0);
    if ((threadIdx.x & 31) == 0 && v < V) vbits[v >> 5] = word;
  }
}

// One thread per edge slot, a CTA per tile of kRecTile consecutive slots.  The source vertex of a
// slot is found in two levels: two threads bisect the whole offset array for the tile's first and
// last slot, the offsets of the vertices in between are copied to shared memory (a tile of 2048
// slots spans 75 vertices on average on the R-MAT graphs, empty ones included), and every thread
// bisects that copy.  A tile that spans more vertices than the copy holds (long runs of empty
// vertices) bisects the global array inside the tile's vertex range instead.
constexpr u32 kRecTile = 2048, kRecSpan = 4096;
__device__ __forceinline__ u32 last_vertex_at_or_before(const u32* __restrict__ xadj, u32 lo, u32 hi, u32 e) {
  while (lo < hi) {  // last v in [lo, hi] with xadj[v] <= e
    const u32 mid = lo + ((hi - lo + 1) >> 1);
    if (__ldg(xadj + mid) <= e) lo = mid;
    else hi = mid - 1;
  }
  return lo;
}
__global__ void __launch_bounds__(256) walk_records_kernel(const u32* __restrict__ xadj,
                                                           const u32* __restrict__ adjncy,
                                                           const Slot* __restrict__ slots,
                                                           const uint2* __restrict__ vinfo, u32 V,
                                                           u64 E, WalkRecord* __restrict__ rec,
                                                           u32* __restrict__ err) {
  __shared__ u32 s_x[kRecSpan + 1];
  __shared__ u32 s_v[2];
  const u64 tiles = (E + kRecTile - 1) / kRecTile;
  for (u64 tile = blockIdx.x; tile < tiles; tile += gridDim.x) {
    const u64 e0 = tile * kRecTile;
    const u64 e1 = e0 + kRecTile < E ? e0 + kRecTile : E;
    if (threadIdx.x < 2)
      s_v[threadIdx.x] = last_vertex_at_or_before(xadj, 0, V - 1, threadIdx.x ? (u32)(e1 - 1) : (u32)e0);
    __syncthreads();
    const u32 v0 = s_v[0], v1 = s_v[1];
    const bool staged = v1 - v0 < kRecSpan;
    if (staged)
      for (u32 i = threadIdx.x; i <= v1 - v0 + 1; i += blockDim.x) s_x[i] = __ldg(xadj + v0 + i);
    __syncthreads();
    for (u64 e = e0 + threadIdx.x; e < e1; e += blockDim.x) {
      u32 off, deg;
      if (staged) {
        u32 lo = 0, hi = v1 - v0;
        while (lo < hi) {
          const u32 mid = lo + ((hi - lo + 1) >> 1);
          if (s_x[mid] <= (u32)e) lo = mid;
          else hi = mid - 1;
        }
        off = s_x[lo];
        deg = s_x[lo + 1] - off;
      } else {
        const u32 v = last_vertex_at_or_before(xadj, v0, v1, (u32)e);
        off = __ldg(xadj + v);
        deg = __ldg(xadj + v + 1) - off;
      }
      Slot s = load_slot(slots + e);
      if (s.alias >= deg) {  // a table that does not belong to this graph: keep the read inside the list
        dev_fail(err, DEV_ERR_INDEX, (u32)e, s.alias, 22);
        s.alias = 0;
      }
      const u32 n_self = __ldg(adjncy + e);
      const u32 n_alias = __ldg(adjncy + (u64)off + s.alias);
      uint2 i_self = make_uint2(0u, 0u), i_alias = make_uint2(0u, 0u);
      if (n_self < V && n_alias < V) {
        i_self = __ldg(vinfo + n_self);
        i_alias = __ldg(vinfo + n_alias);
      } else {
        dev_fail(err, DEV_ERR_INDEX, (u32)e, n_self, n_alias);
      }
      uint4 a, b;
      a.x = __float_as_uint(s.prob);
      a.y = n_self;
      a.z = i_self.x;
      a.w = i_self.y;
      b.x = n_alias;
      b.y = i_alias.x;
      b.z = i_alias.y;
      b.w = s.alias;
      uint4* out = reinterpret_cast<uint4*>(rec + e);
      out[0] = a;
      out[1] = b;
    }
    __syncthreads();
  }
}

struct RecordWalkArgs {
  const WalkRecord* rec;
  const uint2* vinfo;
  const u32* vbits;
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
  float tp;
  u32 unbiased;  // uniform neighbour: the column's own neighbour is always kept (SKW_WALK_UNBIASED)
};

// Same lane-owns-a-stride loop as walk_offline_kernel; a step is one record load.
template <int APP>
__global__ void __launch_bounds__(256) walk_records_walk_kernel(const RecordWalkArgs a) {
  const u64 T = (u64)gridDim.x * blockDim.x;
  u64 w = (u64)blockIdx.x * blockDim.x + threadIdx.x;
  u64 edges = 0;
  bool have = w < a.n;
  u32 off = 0, deg = 0, step = 0;
  u32* row = nullptr;
  Rand4 r{0, 0, 0, 0};  // random words of the walker's current step
  auto begin = [&]() {
    const u32 cur = __ldg(a.starts + w);
    row = a.paths + w * a.hop_num;
    row[0] = cur;
    step = 0;
    if (cur >= a.V) {
      dev_fail(a.err, DEV_ERR_INDEX, cur, 0, (u32)w);
      off = 0;
      deg = 0;
    } else if ((__ldg(a.vbits + (cur >> 5)) >> (cur & 31)) & 1u) {
      const uint2 vi = ldg_once(a.vinfo + cur);
      off = vi.x;
      deg = vi.y;
    } else {
      off = 0;
      deg = 0;
    }
    r = philox_tagged(a.seed, TAG_WALK, a.walker_base + w * a.walker_stride, 0, 0);
  };
  if (have) begin();
  while (have) {
    bool go = step + 1 < a.hop_num && deg != 0;
    if (APP == SKW_APP_PPR && go && u01(r.z) < a.tp) go = false;
    if (go) {
      u32 rw[8];
      load_record(a.rec + (u64)off + __umulhi(r.x, deg), rw);
      // the next step's random words do not depend on the record: computing them here overlaps the
      // load's latency (what a walk is made of when few walkers are in flight)
      const Rand4 rn = philox_tagged(a.seed, TAG_WALK, a.walker_base + w * a.walker_stride, step + 1, 0);
      const bool keep = a.unbiased || u01(r.y) < __uint_as_float(rw[0]);
      ++step;
      row[step] = keep ? rw[1] : rw[4];
      off = keep ? rw[2] : rw[5];
      deg = keep ? rw[3] : rw[6];
      r = rn;
    } else {
      a.lengths[w] = step;
      edges += step;
      w += T;
      have = w < a.n;
      if (have) begin();
    }
  }
  add_edges(a.sum, edges);
}

// PPR over the walk records, one warp per chunk of kChunk consecutive walkers.
//
// Most PPR walks end after a handful of steps, so the loop is dominated by handing lanes their
// next walker.  Set-up: the chunk's start vertices and their {offset, degree} entries are fetched
// up front, independent loads issued together, and parked in per-walker staging rows in shared
// memory (cell 0 = start, cells 1, 2 = offset, degree until the walker's first steps overwrite
// them).  Lanes take walkers from a warp-wide counter (ballot + popc, no atomics) as they become
// free, which costs two shared-memory reads, so the loop holds exactly one dependent global load
// per step.  The first kStage cells of every path are staged in shared memory and written out,
// with the lengths, when the chunk is done (8 lanes per row); cells from kStage on go straight to
// the row.
//
// Measured on B200, 8 M walkers on the scale-26 graph (20.9 M sampled edges per launch): 0.97 ms
// against 1.17 ms for the lane-owns-a-stride kernel; 0.67 ms with the path stores left out, i.e.
// the 8 M isolated row prefixes (one or two 32-byte sectors each, rows hop_num * 4 bytes apart)
// cost DRAM about as much as the record reads, whether they are written step by step or together
// at the end, with default or streaming stores; padding the prefixes to whole 32-byte sectors
// (so that no partly written sector leaves L2) made the launch 12 % slower.  Chunks of 64 walkers
// with 8 warps per CTA were the best of {64, 128, 256} x {4, 8, 16}.
// A batch of 1 M walkers is 1.65 waves of resident CTAs.  Two ways of avoiding the second wave were
// built and compared with this kernel on one GPU, back to back (1 M walkers on the scale-22 graph /
// 8 M on scale 26): chunks handed out from a global atomic cursor to a persistent grid, 0.185 / 0.996 ms
// against 0.174 / 0.973 ms here; chunks of 128 walkers, so that every CTA is resident at once, 0.172 /
// 1.049 ms against 0.173 / 0.971 ms.  Neither helps: the hardware's CTA backfill already keeps the SMs
// loaded, and a small batch is bounded by its longest walks -- with tp = 0.15 the longest of a million
// walks makes 80 to 100 dependent steps, slow ones while the memory system is saturated (300 K lanes in
// flight at 43 G accesses/s are 7 us per access) and 0.6-0.9 us each once it has drained.
constexpr u32 kChunk = 64, kStage = 8;
template <int WARPS, int CHUNK, int STAGE>
__global__ void __launch_bounds__(WARPS * 32, 2048 / (WARPS * 32)) walk_records_ppr_kernel(const RecordWalkArgs a) {
  constexpr u32 kPitch = STAGE + 1;
  __shared__ u32 s_buf[WARPS][CHUNK * kPitch];
  __shared__ uint16_t s_len[WARPS][CHUNK];
  const u32 lane = threadIdx.x & 31, wib = threadIdx.x >> 5;
  const u64 w_begin = ((u64)blockIdx.x * WARPS + wib) * CHUNK;
  if (w_begin >= a.n) return;  // the whole warp leaves; nothing below synchronises the CTA
  const u32 cnt = (u32)min((u64)CHUNK, a.n - w_begin);
  u32* buf = s_buf[wib];
  uint16_t* len = s_len[wib];
  {
    u32 st[CHUNK / 32];
    bool live[CHUNK / 32];
#pragma unroll
    for (int k = 0; k < (int)(CHUNK / 32); ++k) {
      const u32 i = k * 32 + lane;
      st[k] = i < cnt ? __ldg(a.starts + w_begin + i) : 0u;
    }
#pragma unroll
    for (int k = 0; k < (int)(CHUNK / 32); ++k) {
      const u32 i = k * 32 + lane;
      live[k] = false;
      if (i < cnt) {
        if (st[k] >= a.V) dev_fail(a.err, DEV_ERR_INDEX, st[k], 0, (u32)(w_begin + i));
        else live[k] = (__ldg(a.vbits + (st[k] >> 5)) >> (st[k] & 31)) & 1u;
      }
    }
#pragma unroll
    for (int k = 0; k < (int)(CHUNK / 32); ++k) {
      const u32 i = k * 32 + lane;
      uint2 vi = make_uint2(0u, 0u);
      if (live[k]) vi = ldg_once(a.vinfo + st[k]);
      if (i < cnt) {
        buf[i * kPitch] = st[k];
        buf[i * kPitch + 1] = vi.x;
        buf[i * kPitch + 2] = vi.y;
      }
    }
  }
  __syncwarp();
  const u32 lt = (1u << lane) - 1u;
  u32 next = 0;  // walkers of the chunk handed out so far (the same in every lane)
  bool active = false;
  u32 local = 0, off = 0, deg = 0, step = 0;
  u64 edges = 0;
  Rand4 r{0, 0, 0, 0};  // random words of the walker's current step
  for (;;) {
    const u32 need = __ballot_sync(0xFFFFFFFFu, !active);
    if (need && next < cnt) {
      const u32 mine = next + __popc(need & lt);
      if (!active && mine < cnt) {
        local = mine;
        off = buf[local * kPitch + 1];
        deg = buf[local * kPitch + 2];
        step = 0;
        active = true;
        r = philox_tagged(a.seed, TAG_WALK, a.walker_base + (w_begin + local) * a.walker_stride, 0, 0);
      }
      next = min(cnt, next + (u32)__popc(need));
    }
    if (!__any_sync(0xFFFFFFFFu, active)) break;
    if (active) {
      const bool go = step + 1 < a.hop_num && deg != 0 && !(u01(r.z) < a.tp);
      if (go) {
        u32 rw[8];
        load_record(a.rec + (u64)off + __umulhi(r.x, deg), rw);
        // the next step's random words do not depend on the record: computing them here overlaps the
        // load's latency, which is what the end of a pass is made of
        const u32 ry = r.y;
        r = philox_tagged(a.seed, TAG_WALK, a.walker_base + (w_begin + local) * a.walker_stride, step + 1, 0);
        const bool keep = a.unbiased || u01(ry) < __uint_as_float(rw[0]);
        ++step;
        const u32 nv = keep ? rw[1] : rw[4];
        if (step < (u32)STAGE) buf[local * kPitch + step] = nv;
        else a.paths[(w_begin + local) * a.hop_num + step] = nv;
        off = keep ? rw[2] : rw[5];
        deg = keep ? rw[3] : rw[6];
      } else {
        len[local] = (uint16_t)step;
        edges += step;
        active = false;
      }
    }
  }
  __syncwarp();
  // write-out: 8 lanes per row, four neighbouring rows per pass; then the lengths, coalesced
  for (u32 r = lane >> 3; r < cnt; r += 4) {
    const u32 c = lane & 7;
    const u32 cells = min((u32)len[r] + 1u, (u32)STAGE);
    if (c < cells) a.paths[(w_begin + r) * a.hop_num + c] = buf[r * kPitch + c];
  }
  for (u32 i = lane; i < cnt; i += 32) a.lengths[w_begin + i] = len[i];
  add_edges(a.sum, edges);
}

// Copy the written part of every path row (cells 0..length) from the device matrix into a host
// matrix that the GPU can address (pinned memory), 8 lanes per row.  For PPR most rows hold a
// handful of cells, so this moves a few percent of what a copy of the whole matrix would.
__global__ void __launch_bounds__(256) copy_row_prefixes_kernel(const u32* __restrict__ src,
                                                                u32* __restrict__ dst,
                                                                const u32* __restrict__ lengths, u64 n,
                                                                u32 hop_num) {
  const u32 sub = threadIdx.x & 7;
  const u64 rows_per_pass = ((u64)gridDim.x * blockDim.x) >> 3;
  for (u64 w = ((u64)blockIdx.x * blockDim.x + threadIdx.x) >> 3; w < n; w += rows_per_pass) {
    const u32 cells = min(__ldg(lengths + w) + 1u, hop_num);
    const u32* s = src + w * hop_num;
    u32* d = dst + w * hop_num;
    for (u32 c = sub; c < cells; c += 8) d[c] = s[c];
  }
}

// Packed result: the written cells of row w (0..length) go to packed[offs[w] ..), rows back to
// back in walker order; 8 lanes per row, so neighbouring rows fill whole sectors of the output.
struct CellsOfRow {
  __host__ __device__ u64 operator()(u32 length) const { return (u64)length + 1; }
};

__global__ void __launch_bounds__(256) pack_rows_kernel(const u32* __restrict__ src, u32* __restrict__ packed,
                                                        const u32* __restrict__ lengths,
                                                        const u64* __restrict__ offs, u64 n, u32 hop_num,
                                                        u64 capacity, u64* __restrict__ total,
                                                        uint8_t* __restrict__ lengths8) {
  const u32 sub = threadIdx.x & 7;
  const u64 rows_per_pass = ((u64)gridDim.x * blockDim.x) >> 3;
  for (u64 w = ((u64)blockIdx.x * blockDim.x + threadIdx.x) >> 3; w < n; w += rows_per_pass) {
    const u32 len = __ldg(lengths + w);
    const u32 cells = min(len + 1u, hop_num);
    const u64 o = __ldg(offs + w);
    if (lengths8 && sub == 0) lengths8[w] = (uint8_t)len;  // the caller asked for one byte per walk
    if (w == n - 1 && sub == 0) *total = o + cells;  // cells the whole batch needs
    // rows that do not fit are left out: the host compares *total with the capacity and packs again
    // into a larger buffer
    if (o + cells > capacity) continue;
    const u32* s = src + w * hop_num;
    for (u32 c = sub; c < cells; c += 8) packed[o + c] = ldg_once(s + c);
  }
}

__global__ void __launch_bounds__(256) generate_starts_kernel(u32* __restrict__ starts, u64 n,
                                                              u64 id_base, u64 seed, u32 V) {
  for (u64 i = (u64)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (u64)gridDim.x * blockDim.x) {
    const Rand4 r = philox_tagged(seed, TAG_STRT, id_base + i, 0, 0);
    starts[i] = __umulhi(r.x, V);
  }
}

// Grid of the all-steps walk kernels.  A lane walks its walkers one after another, so a CTA lives
// as long as its unluckiest lane; many short CTAs (about 5 are resident per SM at a time) keep the
// SMs evenly loaded to the end.  Measured on B200 for 1, 2, 4 and 8 M walkers alike: fixed-length
// walks are fastest with one walker per thread (8 M walkers, scale-26 DeepWalk: 6.8 ms against
// 7.4 at three per thread and 10.3 at 8 CTAs per SM); PPR, where most walkers stop after a few
// steps, with three walkers per thread (1.19 ms against 1.35 at one per thread and 1.46 at 8 CTAs
// per SM; PPR over walk records has its own chunked kernel, walk_records_ppr_kernel).
static int walk_grid(uint32_t app, u64 n) {
  const u64 per_cta = 256ull * (app == SKW_APP_PPR ? 3 : 1);
  const u64 b = (n + per_cta - 1) / per_cta;
  return (int)(b ? (b < 0x7FFFFFFFull ? b : 0x7FFFFFFFull) : 1);
}

// Measurement aid: a dependent chain of random 32-byte record loads, the memory behaviour of a walk
// stripped of everything else.  Every thread follows `iters` pseudo-random hops through `nrec`
// records with the same load instruction the record walk uses.
__global__ void __launch_bounds__(256) probe_gather_kernel(const WalkRecord* __restrict__ rec, u64 nrec,
                                                           u32 iters, unsigned long long* __restrict__ sink) {
  const u64 tid = (u64)blockIdx.x * blockDim.x + threadIdx.x;
  u64 cur = (tid * 0x9E3779B97F4A7C15ull) % nrec;
  u32 acc = 0;
  for (u32 it = 0; it < iters; ++it) {
    u32 w[8];
    load_record(rec + cur, w);
    acc += w[0];
    u64 x = cur * 31 + w[7] + it + tid;
    x ^= x >> 33;
    x *= 0xff51afd7ed558ccdull;
    x ^= x >> 33;
    cur = x % nrec;
  }
  if (acc == 0x12345677u) atomicAdd(sink, 1ull);  // keeps the loads alive
}

static int grid_for(const skw_ctx* ctx, u64 n, int per_sm) {
  const u64 want = (n + 255) / 256;
  const u64 cap = (u64)ctx->sm_count * per_sm;
  return (int)(want < cap ? (want ? want : 1) : cap);
}

}  // namespace skw

using namespace skw;

extern "C" {

int skw_generate_starts_device(skw_ctx* ctx, uint64_t n, uint64_t id_base, uint64_t seed,
                               uint32_t* d_starts) {
  if (!ctx || (n && !d_starts)) return SKW_ERR_ARG;
  if (!ctx->V) return fail(ctx, SKW_ERR_STATE, "skw_generate_starts_device: no graph resident");
  DeviceGuard g(ctx->device);
  if (n) {
    generate_starts_kernel<<<grid_for(ctx, n, 8), 256, 0, ctx->stream>>>(d_starts, n, id_base, seed, ctx->V);
    SKW_LAUNCHED(ctx);
  }
  return SKW_OK;
}

int skw_walk_records_build(skw_ctx* ctx, float* ms) {
  if (!ctx) return SKW_ERR_ARG;
  if (!ctx->table_ready) return fail(ctx, SKW_ERR_STATE, "skw_walk_records_build: build or import the alias table first");
  DeviceGuard g(ctx->device);
  ctx->records_ready = false;
  // any failure below leaves no half-built records behind
  auto body = [&]() -> int {
    if (!ctx->records) SKW_CUDA(ctx, cudaMalloc(&ctx->records, sizeof(WalkRecord) * (ctx->E ? ctx->E : 1)));
    if (!ctx->vinfo) SKW_CUDA(ctx, cudaMalloc(&ctx->vinfo, sizeof(uint2) * ((size_t)ctx->V + 1)));
    if (!ctx->vbits) SKW_CUDA(ctx, cudaMalloc(&ctx->vbits, sizeof(u32) * ((size_t)ctx->V / 32 + 1)));
    int rc = err_reset(ctx);
    if (rc != SKW_OK) return rc;
    cudaStream_t st = ctx->stream;
    SKW_CUDA(ctx, cudaEventRecord(ctx->ev0, st));
    if (ctx->V) {
      SKW_CUDA(ctx, cudaMemsetAsync(ctx->d_sum + 3, 0, sizeof(uint64_t), st));
      vertex_info_kernel<<<ctx->sm_count * 16, 256, 0, st>>>(ctx->xadj, ctx->slots, ctx->V,
                                                              static_cast<uint2*>(ctx->vinfo), static_cast<u32*>(ctx->vbits),
                                                              reinterpret_cast<u32*>(ctx->d_sum + 3));
      SKW_LAUNCHED(ctx);
      SKW_CUDA(ctx, cudaMemcpyAsync(ctx->h_sum + 3, ctx->d_sum + 3, sizeof(uint64_t), cudaMemcpyDeviceToHost, st));
    }
    if (ctx->E && ctx->V) {
      const u64 tiles = (ctx->E + kRecTile - 1) / kRecTile;
      const u64 cap = (u64)ctx->sm_count * 32;
      walk_records_kernel<<<(unsigned)(tiles < cap ? tiles : cap), 256, 0, st>>>(
          ctx->xadj, ctx->adjncy, ctx->slots, static_cast<const uint2*>(ctx->vinfo), ctx->V, ctx->E,
          static_cast<WalkRecord*>(ctx->records), ctx->d_err);
      SKW_LAUNCHED(ctx);
    }
    SKW_CUDA(ctx, cudaEventRecord(ctx->ev1, st));
    if ((rc = err_check(ctx, "skw_walk_records_build")) != SKW_OK) return rc;  // synchronises the stream
    if (ms) SKW_CUDA(ctx, cudaEventElapsedTime(ms, ctx->ev0, ctx->ev1));
    return SKW_OK;
  };
  const int rc = body();
  if (rc != SKW_OK) {
    const std::string why = ctx->err;
    cudaGetLastError();
    drop_records(ctx);
    ctx->err = why;
    return rc;
  }
  ctx->records_ready = true;
  // every vertex with out-edges has a usable table: the records' offsets and degrees are then those of
  // the graph itself, and unbiased walks may follow them too
  ctx->records_all_usable = ctx->V == 0 || (ctx->h_sum[3] & 0xFFFFFFFFull) == 0;
  return SKW_OK;
}

int skw_ctx_take_sampled_edges(skw_ctx* ctx, uint64_t* out) {
  if (!ctx) return SKW_ERR_ARG;
  DeviceGuard g(ctx->device);
  SKW_CUDA(ctx, cudaMemcpyAsync(ctx->h_sum + 1, ctx->d_sum + 1, sizeof(uint64_t), cudaMemcpyDeviceToHost, ctx->stream));
  int rc = err_check(ctx, "enqueued walks");  // synchronises the stream
  const uint64_t v = ctx->h_sum[1];
  SKW_CUDA(ctx, cudaMemsetAsync(ctx->d_sum + 1, 0, sizeof(uint64_t), ctx->stream));
  if (rc != SKW_OK) {
    err_reset(ctx);
    return rc;
  }
  if (out) *out = v;
  return SKW_OK;
}

int skw_probe_random_gather(skw_ctx* ctx, uint64_t footprint_bytes, uint32_t iters, double* gaccesses_per_s) {
  if (!ctx || !gaccesses_per_s) return SKW_ERR_ARG;
  if (footprint_bytes < (1ull << 20) || iters == 0)
    return fail(ctx, SKW_ERR_ARG, "skw_probe_random_gather: need a footprint of at least 1 MiB and iters > 0");
  DeviceGuard g(ctx->device);
  const u64 nrec = footprint_bytes / sizeof(WalkRecord);
  WalkRecord* buf = nullptr;
  SKW_CUDA(ctx, cudaMalloc(&buf, nrec * sizeof(WalkRecord)));
  cudaStream_t st = ctx->stream;
  cudaError_t e = cudaMemsetAsync(buf, 1, nrec * sizeof(WalkRecord), st);
  const int grid = ctx->sm_count * 8;
  unsigned long long* sink = reinterpret_cast<unsigned long long*>(ctx->d_sum) + 1;
  float ms = 0;
  if (e == cudaSuccess) {
    probe_gather_kernel<<<grid, 256, 0, st>>>(buf, nrec, 8, sink);  // warm-up
    cudaEventRecord(ctx->ev0, st);
    probe_gather_kernel<<<grid, 256, 0, st>>>(buf, nrec, iters, sink);
    cudaEventRecord(ctx->ev1, st);
    ctx->launches += 2;
    e = cudaStreamSynchronize(st);
    if (e == cudaSuccess) e = cudaEventElapsedTime(&ms, ctx->ev0, ctx->ev1);
  }
  cudaFree(buf);
  if (e != cudaSuccess) return fail_cuda(ctx, e, "skw_probe_random_gather", __FILE__, __LINE__);
  *gaccesses_per_s = (double)grid * 256.0 * iters / (ms * 1e-3) / 1e9;
  return SKW_OK;
}

int skw_walk_records_free(skw_ctx* ctx) {
  if (!ctx) return SKW_ERR_ARG;
  DeviceGuard g(ctx->device);
  SKW_CUDA(ctx, cudaStreamSynchronize(ctx->stream));
  cudaFree(ctx->records);
  cudaFree(ctx->vinfo);
  cudaFree(ctx->vbits);
  ctx->records = nullptr;
  ctx->vinfo = nullptr;
  ctx->vbits = nullptr;
  ctx->records_ready = false;
  return SKW_OK;
}

// Argument and state checks shared by the walk entry points.
static int walk_check(skw_ctx* ctx, const skw_walk_params* prm) {
  if (prm->hop_num < 1) return fail(ctx, SKW_ERR_ARG, "skw_walk: hop_num must be >= 1");
  if (prm->app > SKW_APP_NODE2VEC) return fail(ctx, SKW_ERR_ARG, "skw_walk: unknown app %u", prm->app);
  if (prm->mode > SKW_MODE_ONLINE) return fail(ctx, SKW_ERR_ARG, "skw_walk: unknown mode %u", prm->mode);
  if (prm->app == SKW_APP_PPR && !(prm->tp >= 0.0f && prm->tp <= 1.0f))
    return fail(ctx, SKW_ERR_ARG, "skw_walk: tp must be in [0,1]");
  if (prm->app == SKW_APP_NODE2VEC && !(prm->p > 0.0f && prm->q > 0.0f))
    return fail(ctx, SKW_ERR_ARG, "skw_walk: p and q must be positive");
  if (!ctx->xadj) return fail(ctx, SKW_ERR_STATE, "skw_walk: no graph resident");
  const bool unbiased = (prm->flags & SKW_WALK_UNBIASED) != 0;
  const bool online = prm->mode == SKW_MODE_ONLINE && !unbiased;
  if (!online && !unbiased && !ctx->table_ready)
    return fail(ctx, SKW_ERR_STATE, "skw_walk: offline mode needs skw_alias_build_offline or skw_alias_import first");
  if (online && !ctx->adjwgt) return fail(ctx, SKW_ERR_STATE, "skw_walk: online mode needs the edge weights");
  return SKW_OK;
}

// Queue the kernels of one batch of walkers on the context's stream; sampled edges are added to *sum.
// No reset, no readback, no synchronisation (the online table path allocates on first use).
static int walk_launch(skw_ctx* ctx, const skw_walk_params* prm, const uint32_t* d_starts, uint64_t n,
                       uint32_t* d_paths, uint32_t* d_lengths, unsigned long long* sum) {
  const bool unbiased = (prm->flags & SKW_WALK_UNBIASED) != 0;
  const bool online = prm->mode == SKW_MODE_ONLINE && !unbiased;
  int rc;
  // Online walks evaluate the slot they draw straight from the weights; on request they build the
  // tables of the frontier at every step instead (same walks).  With the per-vertex memo and the
  // prefix checkpoints a slot evaluation costs two or three tiles of weights whatever the degree,
  // while a table costs its whole list once per distinct frontier vertex and step, so the direct path
  // is the default for every batch shape.
  bool build_tables = false;
  if (online) build_tables = (prm->flags & (SKW_WALK_CACHE_TABLES | SKW_WALK_BUILD_TABLES)) != 0;
  if (build_tables) {
    drop_records(ctx);  // online builds overwrite table slots
    if ((rc = alloc_table(ctx)) != SKW_OK) return rc;
  }
  if (!n) return SKW_OK;
  WalkArgs a;
  a.xadj = ctx->xadj;
  a.adjncy = ctx->adjncy;
  a.slots = ctx->slots;
  a.starts = d_starts;
  a.paths = d_paths;
  a.lengths = d_lengths;
  a.sum = sum;
  a.err = ctx->d_err;
  a.n = n;
  a.seed = prm->seed;
  a.walker_base = prm->walker_base;
  a.walker_stride = prm->walker_stride ? prm->walker_stride : 1;
  a.V = ctx->V;
  a.hop_num = prm->hop_num;
  a.unbiased = unbiased ? 1u : 0u;
  a.tp = prm->tp;
  a.inv_p = prm->app == SKW_APP_NODE2VEC ? 1.0f / prm->p : 1.0f;
  a.inv_q = prm->app == SKW_APP_NODE2VEC ? 1.0f / prm->q : 1.0f;
  a.fmax = fmaxf(1.0f, fmaxf(a.inv_p, a.inv_q));
  cudaStream_t st = ctx->stream;
  // Walk records serve unbiased walks as well (the record of column c names the c-th neighbour with its
  // offset and degree: one access per step instead of two), as long as every vertex with out-edges has
  // a usable table, i.e. the degrees in the records are the graph's own.
  if (!online && ctx->records_ready && prm->app != SKW_APP_NODE2VEC && (!unbiased || ctx->records_all_usable)) {
    RecordWalkArgs ra;
    ra.unbiased = unbiased ? 1u : 0u;
    ra.rec = static_cast<const WalkRecord*>(ctx->records);
    ra.vinfo = static_cast<const uint2*>(ctx->vinfo);
    ra.vbits = static_cast<const u32*>(ctx->vbits);
    ra.starts = d_starts;
    ra.paths = d_paths;
    ra.lengths = d_lengths;
    ra.sum = a.sum;
    ra.err = a.err;
    ra.n = n;
    ra.seed = a.seed;
    ra.walker_base = a.walker_base;
    ra.walker_stride = a.walker_stride;
    ra.V = a.V;
    ra.hop_num = a.hop_num;
    ra.tp = a.tp;
    const int grid = walk_grid(prm->app, n);
    // (the chunked kernel stages lengths as 16-bit values and has no grid-stride loop)
    const u64 ctas = (n + 8 * kChunk - 1) / (8 * kChunk);
    if (prm->app == SKW_APP_PPR && prm->hop_num <= 65535 && ctas <= 0x7FFFFFFFull) {
      walk_records_ppr_kernel<8, kChunk, kStage><<<(unsigned)ctas, 256, 0, st>>>(ra);
    } else if (prm->app == SKW_APP_PPR) walk_records_walk_kernel<SKW_APP_PPR><<<grid, 256, 0, st>>>(ra);
    else walk_records_walk_kernel<SKW_APP_DEEPWALK><<<grid, 256, 0, st>>>(ra);
    SKW_LAUNCHED(ctx);
  } else if (!online) {
    const int grid = walk_grid(prm->app, n);
    switch (prm->app) {
      case SKW_APP_DEEPWALK: walk_offline_kernel<SKW_APP_DEEPWALK><<<grid, 256, 0, st>>>(a); break;
      case SKW_APP_PPR: walk_offline_kernel<SKW_APP_PPR><<<grid, 256, 0, st>>>(a); break;
      default: walk_offline_kernel<SKW_APP_NODE2VEC><<<grid, 256, 0, st>>>(a); break;
    }
    SKW_LAUNCHED(ctx);
  } else if (!build_tables) {
    if ((rc = launch_walk_online_direct(ctx, a, prm->app)) != SKW_OK) return rc;
  } else {
    const int grid = grid_for(ctx, n, 8);
    walk_online_init_kernel<<<grid, 256, 0, st>>>(a);
    SKW_LAUNCHED(ctx);
    for (uint32_t step = 0; step + 1 < prm->hop_num; ++step) {
      if ((rc = frontier_collect(ctx, d_paths, n, 1, prm->hop_num, step, d_lengths,
                                 step == 0 || !(prm->flags & SKW_WALK_CACHE_TABLES))) != SKW_OK) return rc;
      switch (prm->app) {
        case SKW_APP_DEEPWALK: walk_online_step_kernel<SKW_APP_DEEPWALK><<<grid, 256, 0, st>>>(a, step); break;
        case SKW_APP_PPR: walk_online_step_kernel<SKW_APP_PPR><<<grid, 256, 0, st>>>(a, step); break;
        default: walk_online_step_kernel<SKW_APP_NODE2VEC><<<grid, 256, 0, st>>>(a, step); break;
      }
      SKW_LAUNCHED(ctx);
    }
  }
  return SKW_OK;
}

int skw_walk_device(skw_ctx* ctx, const skw_walk_params* prm, const uint32_t* d_starts, uint64_t n,
                    uint32_t* d_paths, uint32_t* d_lengths, float* ms, uint64_t* sampled_edges) {
  if (!ctx || !prm) return SKW_ERR_ARG;
  if (n && (!d_starts || !d_paths || !d_lengths))
    return fail(ctx, SKW_ERR_ARG, "skw_walk: null buffer");
  int rc = walk_check(ctx, prm);
  if (rc != SKW_OK) return rc;
  DeviceGuard g(ctx->device);
  cudaStream_t st = ctx->stream;
  // With both result pointers null the call only enqueues work: no reset, no readback, no
  // synchronisation.  Sampled edges then add up in a second counter and a device error stays
  // recorded until skw_ctx_take_sampled_edges() (or a later synchronous call) looks at it.
  const bool enqueue_only = !ms && !sampled_edges;
  unsigned long long* sum = reinterpret_cast<unsigned long long*>(ctx->d_sum) + (enqueue_only ? 1 : 0);
  if (!enqueue_only) {
    if ((rc = err_reset(ctx)) != SKW_OK) return rc;
    SKW_CUDA(ctx, cudaMemsetAsync(ctx->d_sum, 0, sizeof(uint64_t), st));
    SKW_CUDA(ctx, cudaEventRecord(ctx->ev0, st));
  }
  if ((rc = walk_launch(ctx, prm, d_starts, n, d_paths, d_lengths, sum)) != SKW_OK) return rc;
  if (enqueue_only) return SKW_OK;
  SKW_CUDA(ctx, cudaEventRecord(ctx->ev1, st));
  SKW_CUDA(ctx, cudaMemcpyAsync(ctx->h_sum, ctx->d_sum, sizeof(uint64_t), cudaMemcpyDeviceToHost, st));
  if ((rc = err_check(ctx, "skw_walk")) != SKW_OK) return rc;
  if (ms) SKW_CUDA(ctx, cudaEventElapsedTime(ms, ctx->ev0, ctx->ev1));
  if (sampled_edges) *sampled_edges = *ctx->h_sum;
  return SKW_OK;
}

// Large batches into the caller's n x hop_num host matrix: the walks come home packed (contiguous
// copies, only cells that hold a vertex cross the bus) into pinned staging owned by the context, and
// host threads scatter them into the rows.  A kernel writing row prefixes straight into mapped host
// memory sends one small bus write per row (8 M PPR rows: 22 ms); a copy of the whole matrix moves
// every unused cell as well.  Cells past a walk's end keep what the caller had there.
static int walk_rows_by_scatter(skw_ctx* ctx, const skw_walk_params* prm, const uint32_t* h_starts, uint64_t n,
                                uint32_t* h_paths, uint32_t* h_lengths, float* ms, uint64_t* sampled_edges) {
  const uint64_t full = n * prm->hop_num;
  uint64_t want = full;
  if (prm->app == SKW_APP_PPR && prm->tp > 0.0f)
    want = std::min<uint64_t>(full, (uint64_t)((double)n * (1.0 / prm->tp + 2.0)) + 4096);
  uint64_t cells = 0;
  for (int attempt = 0; attempt < 2; ++attempt) {
    if (ctx->h_pack_cells < want) {
      if (ctx->h_pack) cudaFreeHost(ctx->h_pack);
      ctx->h_pack = nullptr;
      ctx->h_pack_cells = 0;
      SKW_CUDA(ctx, cudaMallocHost(&ctx->h_pack, sizeof(uint32_t) * (size_t)want));
      ctx->h_pack_cells = want;
    }
    const int rc = skw_walk_packed(ctx, prm, h_starts, n, ctx->h_pack, ctx->h_pack_cells, h_lengths, &cells, ms,
                                   sampled_edges);
    if (rc == SKW_OK) break;
    if (rc != SKW_ERR_ARG || cells <= ctx->h_pack_cells || attempt == 1) return rc;
    want = std::min<uint64_t>(full, cells + (cells >> 3) + 4096);  // the staging was too small: once more
  }
  if (!ctx->host_pool) {
    unsigned hc = std::thread::hardware_concurrency();
    ctx->host_pool = new HostPool((int)std::min<unsigned>(hc ? hc : 1u, 32u));
  }
  HostPool* pool = static_cast<HostPool*>(ctx->host_pool);
  const int T = pool->size();
  std::vector<uint64_t> first(T + 1, 0);  // cells before each thread's block of walkers
  const uint32_t hop = prm->hop_num;
  pool->run([&](int t, int) {
    const uint64_t lo = n * t / T, hi = n * (t + 1) / T;
    uint64_t sum = 0;
    for (uint64_t w = lo; w < hi; ++w) sum += (uint64_t)std::min<uint32_t>(h_lengths[w] + 1u, hop);
    first[t + 1] = sum;
  });
  for (int t = 0; t < T; ++t) first[t + 1] += first[t];
  if (first[T] != cells)
    return fail(ctx, SKW_ERR_DEVICE, "skw_walk: packed result holds %llu cells, the lengths add up to %llu",
                (unsigned long long)cells, (unsigned long long)first[T]);
  const uint32_t* packed = ctx->h_pack;
  pool->run([&](int t, int) {
    const uint64_t lo = n * t / T, hi = n * (t + 1) / T;
    uint64_t o = first[t];
    // every row is a cache miss of its own (rows lie hop_num cells apart): ask for the lines a few rows
    // ahead, and copy short rows cell by cell (most PPR rows hold a handful of cells)
    constexpr uint64_t kAhead = 24;
    for (uint64_t w = lo; w < hi; ++w) {
      if (w + kAhead < hi) __builtin_prefetch(h_paths + (w + kAhead) * hop, 1, 0);
      const uint32_t c = std::min<uint32_t>(h_lengths[w] + 1u, hop);
      uint32_t* row = h_paths + w * hop;
      const uint32_t* src = packed + o;
      if (c <= 8) {
        for (uint32_t k = 0; k < c; ++k) row[k] = src[k];
      } else {
        memcpy(row, src, sizeof(uint32_t) * c);
      }
      o += c;
    }
  });
  return SKW_OK;
}

int skw_walk(skw_ctx* ctx, const skw_walk_params* prm, const uint32_t* h_starts, uint64_t n,
             uint32_t* h_paths, uint32_t* h_lengths, float* ms, uint64_t* sampled_edges) {
  if (!ctx || !prm) return SKW_ERR_ARG;
  if (n && (!h_starts || !h_paths || !h_lengths)) return fail(ctx, SKW_ERR_ARG, "skw_walk: null buffer");
  if (prm->hop_num < 1) return fail(ctx, SKW_ERR_ARG, "skw_walk: hop_num must be >= 1");
  DeviceGuard g(ctx->device);
  if (n >= (1u << 18)) return walk_rows_by_scatter(ctx, prm, h_starts, n, h_paths, h_lengths, ms, sampled_edges);
  int rc;
  const size_t nb = sizeof(uint32_t) * (size_t)n;
  if ((rc = ensure_bytes(ctx, &ctx->stage[0], &ctx->stage_bytes[0], nb)) != SKW_OK) return rc;
  if ((rc = ensure_bytes(ctx, &ctx->stage[1], &ctx->stage_bytes[1], nb * prm->hop_num)) != SKW_OK) return rc;
  if ((rc = ensure_bytes(ctx, &ctx->stage[2], &ctx->stage_bytes[2], nb)) != SKW_OK) return rc;
  if (n) SKW_CUDA(ctx, cudaMemcpyAsync(ctx->stage[0], h_starts, nb, cudaMemcpyHostToDevice, ctx->stream));
  rc = skw_walk_device(ctx, prm, static_cast<uint32_t*>(ctx->stage[0]), n,
                       static_cast<uint32_t*>(ctx->stage[1]), static_cast<uint32_t*>(ctx->stage[2]), ms,
                       sampled_edges);
  if (rc != SKW_OK) return rc;
  if (n) {
    // Pinned host memory is addressable by the GPU: write only the cells each walk produced.
    // Pageable memory gets the whole matrix (cells past a walk's end then hold stale values).
    cudaPointerAttributes at;
    u32* mapped = nullptr;
    if (cudaPointerGetAttributes(&at, h_paths) == cudaSuccess && at.type == cudaMemoryTypeHost && at.devicePointer)
      mapped = static_cast<u32*>(at.devicePointer);
    else
      cudaGetLastError();
    if (mapped) {
      copy_row_prefixes_kernel<<<ctx->sm_count * 8, 256, 0, ctx->stream>>>(
          static_cast<const u32*>(ctx->stage[1]), mapped, static_cast<const u32*>(ctx->stage[2]), n, prm->hop_num);
      SKW_LAUNCHED(ctx);
    } else {
      SKW_CUDA(ctx, cudaMemcpyAsync(h_paths, ctx->stage[1], nb * prm->hop_num, cudaMemcpyDeviceToHost, ctx->stream));
    }
    SKW_CUDA(ctx, cudaMemcpyAsync(h_lengths, ctx->stage[2], nb, cudaMemcpyDeviceToHost, ctx->stream));
  }
  SKW_CUDA(ctx, cudaStreamSynchronize(ctx->stream));
  return SKW_OK;
}

}  // extern "C"

// The packed host entry points: lengths come home as 32-bit words (h_lengths) or, for walks of at
// most 256 vertices, as bytes (h_lengths8); exactly one of the two is given.
static int walk_packed_impl(skw_ctx* ctx, const skw_walk_params* prm, const uint32_t* h_starts, uint64_t n,
                            uint32_t* h_packed, uint64_t capacity_cells, uint32_t* h_lengths,
                            uint8_t* h_lengths8, uint64_t* cells, float* ms, uint64_t* sampled_edges) {
  if (!ctx || !prm) return SKW_ERR_ARG;
  if (!cells) return fail(ctx, SKW_ERR_ARG, "skw_walk_packed: cells must not be null");
  *cells = 0;
  if (ms) *ms = 0;
  if (sampled_edges) *sampled_edges = 0;
  if (n && (!h_starts || (!h_lengths && !h_lengths8))) return fail(ctx, SKW_ERR_ARG, "skw_walk_packed: null buffer");
  int rc = walk_check(ctx, prm);
  if (rc != SKW_OK) return rc;
  if (h_lengths8 && prm->hop_num > 256)
    return fail(ctx, SKW_ERR_ARG, "skw_walk_packed_u8: a length of up to %u does not fit a byte", prm->hop_num - 1);
  if (!n) return SKW_OK;
  DeviceGuard g(ctx->device);
  cudaStream_t st = ctx->stream, side = ctx->side_stream;
  // Large batches run as up to eight slices.  Everything a slice needs on the device (walk, prefix sum
  // of its row sizes, packing) is queued for ALL slices before the host waits for anything; the side
  // stream brings each slice's cell count, lengths and packed rows home as soon as they exist, while
  // the context's stream is already walking the next slice (the bus carries both directions at once).
  // Walker ids, hence walks, do not depend on the slicing.
  const uint64_t kSliceMin = 1u << 19;
  const uint32_t slices = n >= 8 * kSliceMin ? 8 : (n >= 4 * kSliceMin ? 4 : (n >= 2 * kSliceMin ? 2 : 1));
  static_assert(skw_ctx::kPackSlices >= 8 && skw_ctx::kStages >= 4 + 8, "one event set and one packing buffer per slice");
  // Slice sizes in the ratio 1 : 2 : 4 : 4 ...: the first results are on the bus early (the call is
  // as long as the time to the first packed slice plus the copy of everything), the later slices are
  // large enough to walk efficiently.
  uint64_t base_of[skw_ctx::kPackSlices + 1] = {};
  uint64_t per = n;  // the largest slice
  if (slices > 1) {
    const uint64_t parts = 3 + 4ull * (slices - 2);
    const uint64_t unit = ((n + parts - 1) / parts + 1023) & ~1023ull;
    per = (slices == 2 ? 2 : 4) * unit;
    for (uint32_t c = 0; c <= slices; ++c) {
      const uint64_t b = c == 0 ? 0 : (c == 1 ? unit : (3 + 4ull * (c - 2)) * unit);
      base_of[c] = std::min<uint64_t>(b, n);
    }
  } else {
    base_of[1] = n;
  }
  const uint64_t stride = prm->walker_stride ? prm->walker_stride : 1;
  const size_t offs_bytes = (sizeof(u64) * (size_t)per + 255) & ~(size_t)255;
  size_t tmp_bytes = 0;
  {
    cub::TransformInputIterator<u64, CellsOfRow, const u32*> probe(static_cast<const u32*>(nullptr), CellsOfRow());
    SKW_CUDA(ctx, cub::DeviceScan::ExclusiveSum(nullptr, tmp_bytes, probe, (u64*)nullptr, (long long)per, st));
  }
  if ((rc = ensure_bytes(ctx, &ctx->stage[0], &ctx->stage_bytes[0], sizeof(u32) * (size_t)n)) != SKW_OK) return rc;
  if ((rc = ensure_bytes(ctx, &ctx->stage[1], &ctx->stage_bytes[1], sizeof(u32) * (size_t)n * prm->hop_num)) != SKW_OK)
    return rc;
  if ((rc = ensure_bytes(ctx, &ctx->stage[2], &ctx->stage_bytes[2], sizeof(u32) * (size_t)n)) != SKW_OK) return rc;
  if ((rc = ensure_bytes(ctx, &ctx->stage[3], &ctx->stage_bytes[3], offs_bytes + tmp_bytes)) != SKW_OK) return rc;
  constexpr int kLen8Stage = 4 + skw_ctx::kPackSlices;
  static_assert(skw_ctx::kStages > kLen8Stage, "one more staging buffer for byte lengths");
  if (h_lengths8 && (rc = ensure_bytes(ctx, &ctx->stage[kLen8Stage], &ctx->stage_bytes[kLen8Stage], (size_t)n)) != SKW_OK)
    return rc;
  uint8_t* d_len8 = h_lengths8 ? static_cast<uint8_t*>(ctx->stage[kLen8Stage]) : nullptr;
  u32* d_starts = static_cast<u32*>(ctx->stage[0]);
  u32* d_rows = static_cast<u32*>(ctx->stage[1]);
  u32* d_len = static_cast<u32*>(ctx->stage[2]);
  u64* d_offs = static_cast<u64*>(ctx->stage[3]);
  // Packing buffers, one per slice.  The size of a result changes from call to call (another seed,
  // other lengths), so a buffer that exists is kept as it is and only a result that outgrows it makes
  // it grow (by an eighth more than needed): steady-state calls do not allocate.  First guess: every
  // walk at full length, or the expected PPR length with room to spare.
  uint64_t cap[skw_ctx::kPackSlices] = {}, nc_of[skw_ctx::kPackSlices] = {};
  for (uint32_t c = 0; c < slices; ++c) {
    const uint64_t base = base_of[c];
    if (base >= n) break;
    const uint64_t nc = base_of[c + 1] - base;
    nc_of[c] = nc;
    const uint64_t full = nc * prm->hop_num;
    uint64_t guess = full;
    if (prm->app == SKW_APP_PPR && prm->tp > 0.0f)
      guess = std::min<uint64_t>(full, (uint64_t)((double)nc * (1.0 / prm->tp + 2.0)) + 4096);
    if (ctx->stage[4 + c] && ctx->stage_bytes[4 + c] >= sizeof(u32) * 1024) guess = ctx->stage_bytes[4 + c] / sizeof(u32);
    if ((rc = ensure_bytes(ctx, &ctx->stage[4 + c], &ctx->stage_bytes[4 + c], sizeof(u32) * (size_t)guess)) != SKW_OK) return rc;
    cap[c] = std::min<uint64_t>(ctx->stage_bytes[4 + c] / sizeof(u32), full);
  }
  if ((rc = err_reset(ctx)) != SKW_OK) return rc;
  unsigned long long* scratch_sum = reinterpret_cast<unsigned long long*>(ctx->d_sum) + 2;
  auto scan_and_pack = [&](uint32_t c) -> int {
    const uint64_t base = base_of[c], nc = nc_of[c];
    cub::TransformInputIterator<u64, CellsOfRow, const u32*> row_cells(d_len + base, CellsOfRow());
    size_t tb = tmp_bytes;
    SKW_CUDA(ctx, cub::DeviceScan::ExclusiveSum(reinterpret_cast<char*>(d_offs) + offs_bytes, tb, row_cells, d_offs,
                                                (long long)nc, st));
    SKW_LAUNCHED(ctx);
    // Packed on the device, then one contiguous copy per slice: measured on B200 with 8 M PPR walks,
    // half the time of a pack kernel that writes the pinned host buffer itself (its 4-byte stores
    // per row do not merge into full-size bus writes).
    pack_rows_kernel<<<grid_for(ctx, nc * 8, 8), 256, 0, st>>>(d_rows + base * prm->hop_num,
                                                              static_cast<u32*>(ctx->stage[4 + c]), d_len + base, d_offs, nc,
                                                              prm->hop_num, cap[c], ctx->d_tot + c,
                                                              d_len8 ? d_len8 + base : nullptr);
    SKW_LAUNCHED(ctx);
    SKW_CUDA(ctx, cudaEventRecord(ctx->pk_ready[c], st));
    SKW_CUDA(ctx, cudaStreamWaitEvent(side, ctx->pk_ready[c], 0));
    SKW_CUDA(ctx, cudaMemcpyAsync(ctx->h_tot + c, ctx->d_tot + c, sizeof(u64), cudaMemcpyDeviceToHost, side));
    SKW_CUDA(ctx, cudaEventRecord(ctx->pk_tot[c], side));
    return SKW_OK;
  };
  auto body = [&]() -> int {
    // the start vertices come in slice by slice on the side stream, ahead of everything else it will
    // carry: a walk waits for its own slice only, and no walk waits behind a copy of a later slice
    for (uint32_t c = 0; c < slices && nc_of[c]; ++c) {
      const uint64_t base = base_of[c], nc = nc_of[c];
      SKW_CUDA(ctx, cudaMemcpyAsync(d_starts + base, h_starts + base, sizeof(u32) * (size_t)nc, cudaMemcpyHostToDevice, side));
      SKW_CUDA(ctx, cudaEventRecord(ctx->pk_in[c], side));
    }
    for (uint32_t c = 0; c < slices && nc_of[c]; ++c) {
      const uint64_t base = base_of[c], nc = nc_of[c];
      SKW_CUDA(ctx, cudaStreamWaitEvent(st, ctx->pk_in[c], 0));
      skw_walk_params p = *prm;
      p.walker_base = prm->walker_base + base * stride;
      SKW_CUDA(ctx, cudaEventRecord(ctx->pk_t0[c], st));
      int r = walk_launch(ctx, &p, d_starts + base, nc, d_rows + base * prm->hop_num, d_len + base, scratch_sum);
      if (r != SKW_OK) return r;
      SKW_CUDA(ctx, cudaEventRecord(ctx->pk_t1[c], st));
      if ((r = scan_and_pack(c)) != SKW_OK) return r;
      if (h_lengths8)
        SKW_CUDA(ctx, cudaMemcpyAsync(h_lengths8 + base, d_len8 + base, (size_t)nc, cudaMemcpyDeviceToHost, side));
      else
        SKW_CUDA(ctx, cudaMemcpyAsync(h_lengths + base, d_len + base, sizeof(u32) * (size_t)nc, cudaMemcpyDeviceToHost, side));
    }
    // the host follows the device slice by slice: learn the size, start the copy
    uint64_t total_cells = 0;
    bool fits = h_packed != nullptr;
    float total_ms = 0;
    for (uint32_t c = 0; c < slices && nc_of[c]; ++c) {
      SKW_CUDA(ctx, cudaEventSynchronize(ctx->pk_tot[c]));
      uint64_t slice_cells = ctx->h_tot[c];
      if (fits && total_cells + slice_cells > capacity_cells) fits = false;  // keep going: the caller gets the size
      if (fits && slice_cells > cap[c]) {
        // this slice outgrew its packing buffer: grow it and pack once more (its rows and lengths are
        // still on the device).  Growing frees the old buffer, which waits for the device.
        const uint64_t roomy = std::min<uint64_t>(slice_cells + (slice_cells >> 3) + 4096, nc_of[c] * prm->hop_num);
        int r = ensure_bytes(ctx, &ctx->stage[4 + c], &ctx->stage_bytes[4 + c], sizeof(u32) * (size_t)roomy);
        if (r != SKW_OK) return r;
        cap[c] = roomy;
        if ((r = scan_and_pack(c)) != SKW_OK) return r;
        SKW_CUDA(ctx, cudaEventSynchronize(ctx->pk_tot[c]));
        slice_cells = ctx->h_tot[c];
      }
      if (fits) {
        // on a stream of its own: the side stream already holds the (still waiting) count and length
        // copies of the later slices, and this copy must not queue up behind them
        SKW_CUDA(ctx, cudaStreamWaitEvent(ctx->copy_stream, ctx->pk_ready[c], 0));
        SKW_CUDA(ctx, cudaMemcpyAsync(h_packed + total_cells, ctx->stage[4 + c], sizeof(u32) * (size_t)slice_cells,
                                      cudaMemcpyDeviceToHost, ctx->copy_stream));
      }
      total_cells += slice_cells;
      float t = 0;
      SKW_CUDA(ctx, cudaEventElapsedTime(&t, ctx->pk_t0[c], ctx->pk_t1[c]));  // the walk is long over
      total_ms += t;
    }
    SKW_CUDA(ctx, cudaStreamSynchronize(side));
    SKW_CUDA(ctx, cudaStreamSynchronize(ctx->copy_stream));
    int r = err_check(ctx, "skw_walk_packed");  // synchronises the context's stream
    if (r != SKW_OK) return r;
    *cells = total_cells;
    if (ms) *ms = total_ms;
    if (sampled_edges) *sampled_edges = total_cells - n;  // every walk holds its start plus one vertex per sampled edge
    if (!fits)
      return fail(ctx, SKW_ERR_ARG, "skw_walk_packed: the result needs %llu cells, the buffer holds %llu",
                  (unsigned long long)total_cells, (unsigned long long)(h_packed ? capacity_cells : 0));
    return SKW_OK;
  };
  rc = body();
  if (rc != SKW_OK && rc != SKW_ERR_ARG) {  // leave nothing in flight that still writes the caller's buffers
    const std::string why = ctx->err;
    cudaStreamSynchronize(side);
    cudaStreamSynchronize(ctx->copy_stream);
    cudaStreamSynchronize(st);
    ctx->err = why;
  }
  return rc;
}

extern "C" {

int skw_walk_packed(skw_ctx* ctx, const skw_walk_params* prm, const uint32_t* h_starts, uint64_t n,
                    uint32_t* h_packed, uint64_t capacity_cells, uint32_t* h_lengths, uint64_t* cells,
                    float* ms, uint64_t* sampled_edges) {
  if (ctx && n && !h_lengths) return fail(ctx, SKW_ERR_ARG, "skw_walk_packed: null buffer");
  return walk_packed_impl(ctx, prm, h_starts, n, h_packed, capacity_cells, h_lengths, nullptr, cells, ms,
                          sampled_edges);
}

int skw_walk_packed_u8(skw_ctx* ctx, const skw_walk_params* prm, const uint32_t* h_starts, uint64_t n,
                       uint32_t* h_packed, uint64_t capacity_cells, uint8_t* h_lengths8, uint64_t* cells,
                       float* ms, uint64_t* sampled_edges) {
  if (ctx && n && !h_lengths8) return fail(ctx, SKW_ERR_ARG, "skw_walk_packed_u8: null buffer");
  return walk_packed_impl(ctx, prm, h_starts, n, h_packed, capacity_cells, nullptr, h_lengths8, cells, ms,
                          sampled_edges);
}

}  // extern "C"
