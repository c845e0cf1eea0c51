// Online walks without tables: the slot a walker draws is computed from the weight list.
#include <algorithm>

#include "skw_alias_math.cuh"
#include "skw_ctx.h"
#include "skw_walk_common.cuh"

namespace skw {

// ------------------------------------------------------------------ online walk, direct ----
// An online walk draws ONE slot of the table of the vertex it stands on and never looks at that
// table again.  So instead of building the tables of the whole frontier at every step (degree-class
// builders, one launch per class per step, 8 bytes per edge written and read back), one warp per
// walker computes just the slot it drew, straight from the weight list, with the arithmetic of the
// construction rule -- the same (prob, alias) bits the builders would have stored -- and all steps
// of all walkers run in one launch.
//
// Slot p of a list of n weights (masses M_i, bucket C, d = C - M of smalls, x = M - C of larges):
//   small p:  prob = M_p / C,  alias = first large e (in list order) with X_incl(e) >= D_excl(p)
//   large p:  let k = first small with D_incl(k) > X_incl(p); none: prob = 1, alias = p;
//             else prob = (X_incl(p) + C - D_incl(k)) / C,  alias = first large after p
// where D_* / X_* are the running sums of d over smalls / x over larges.  That takes: the largest
// weight and the total quantised weight (two reductions over the list), a sweep of the masses up
// to p (running sums kept per lane, one reduction at the end) and a second sweep from the start up
// to the crossing.  A sweep handles 128 weights per iteration, 4 consecutive ones per lane, with
// one warp scan for the cumulative quantised weight (and one more in the second sweep).
struct ListPrep {
  u64 W, nC, C;
  double K;
  int B, sh;
};

__device__ __forceinline__ u64 warp_sum_u64(u64 x) {
#pragma unroll
  for (int o = 16; o; o >>= 1) x += __shfl_xor_sync(0xFFFFFFFFu, x, o);
  return x;
}
// exclusive prefix over the lanes; total = sum over the warp
__device__ __forceinline__ u64 warp_excl_u64(u64 x, u32 lane, u64& total) {
  u64 inc = x;
#pragma unroll
  for (int o = 1; o < 32; o <<= 1) {
    const u64 t = __shfl_up_sync(0xFFFFFFFFu, inc, o);
    if (lane >= (u32)o) inc += t;
  }
  total = __shfl_sync(0xFFFFFFFFu, inc, 31);
  return inc - x;
}

// false: the list has no usable weight
__device__ __forceinline__ bool list_prepare(const float* __restrict__ w, u32 n, u32 lane, ListPrep& L) {
  float wmax = 0.0f;
  for (u32 i = lane; i < n; i += 32) wmax = fmaxf(wmax, sane_weight(__ldg(w + i)));
#pragma unroll
  for (int o = 16; o; o >>= 1) wmax = fmaxf(wmax, __shfl_xor_sync(0xFFFFFFFFu, wmax, o));
  if (!(wmax > 0.0f)) return false;
  L.B = bucket_bits(n);
  L.C = (u64)1 << L.B;
  L.sh = weight_shift(wmax, L.B);
  u64 acc = 0;
  for (u32 i = lane; i < n; i += 32) acc += quantise_bits(sane_weight(__ldg(w + i)), L.sh);
  L.W = warp_sum_u64(acc);
  L.nC = (u64)n << L.B;
  L.K = mass_factor(n, L.B, L.W);
  return true;
}

// The largest weight and the total quantised weight of a list depend on the weights only, which do
// not change while a call runs.  For lists of kMemoMinDegree weights and more the first walker that
// stands on a vertex during a call leaves the two numbers in a per-vertex memo (16 bytes, tagged with
// the call's stamp) and later visitors -- the same walker coming back, or others -- read them instead
// of making the two passes over the list again.  Nothing of the table itself is kept: the drawn slot
// is still computed from the weights at every step.  Publication order: values, fence, stamp; a
// reader that sees the stamp fences and then reads the values.
struct PrepMemo {
  u32 stamp;
  float wmax;
  u64 W;
};
constexpr u32 kMemoMinDegree = 256;

// For lists of kCkMinDegree weights and more the same first visit also leaves CHECKPOINTS of two
// prefix sums at every kCkChunk-th list position b (measured on config 3: 19.4 / 17.5 / 16.4 ms per pass
// with chunks of 1024 / 512 / 256 weights and tiles of 128; 11.3 ms with chunks of 128, 8.7 ms with chunks
// and tiles of 64, 8.4 ms with 32, which needs twice the memory again): the cumulative quantised weight Q_b and the
// deficit D_b of the smalls before b (the excess of the larges before b follows from them,
// X_b = D_b + g(Q_b) - b * C).  They are integers and depend on the weights alone, so whoever
// writes them writes the same values.  A later draw of slot p then sweeps the list from the boundary
// before p instead of from its start, and finds the chunk that holds the crossing it looks for by
// bisecting the checkpoints: at most two chunks of weights are visited per step instead of one and a
// half passes over the list, which is what a walk on a power-law graph spends its time on (a walker
// stands on a hub most of the time, and the cost of a draw grows with the hub's degree).  Still no
// slot of a table is kept.  Entry k - 1 of a vertex's checkpoints is boundary k (k >= 1); the vertex
// with first-edge offset `off` owns entries off / kCkChunk ... of one array of E / kCkChunk + 2
// entries (consecutive vertices cannot collide: a list of n weights has (n - 1) / kCkChunk entries).
struct __align__(16) Ckpt {
  u64 Q, D;
};
constexpr u32 kCkChunk = 64, kCkMinDegree = 256;

__device__ void record_checkpoints(const float* __restrict__ w, u32 n, u32 lane, const ListPrep& L, Ckpt* ck);

__device__ __forceinline__ bool list_prepare_memo(const float* __restrict__ w, u32 n, u32 lane, ListPrep& L,
                                                  PrepMemo* __restrict__ memo, u32 stamp, Ckpt* ck) {
  if (memo == nullptr || n < kMemoMinDegree) return list_prepare(w, n, lane, L);
  u32 seen = 0;
  if (lane == 0) seen = *reinterpret_cast<volatile u32*>(&memo->stamp);
  seen = __shfl_sync(0xFFFFFFFFu, seen, 0);
  if (seen == stamp) {
    float wmax = 0.0f;
    u64 W = 0;
    if (lane == 0) {
      __threadfence();
      wmax = *reinterpret_cast<volatile float*>(&memo->wmax);
      W = *reinterpret_cast<volatile u64*>(&memo->W);
    }
    wmax = __shfl_sync(0xFFFFFFFFu, wmax, 0);
    W = __shfl_sync(0xFFFFFFFFu, W, 0);
    if (!(wmax > 0.0f)) return false;
    L.B = bucket_bits(n);
    L.C = (u64)1 << L.B;
    L.sh = weight_shift(wmax, L.B);
    L.W = W;
    L.nC = (u64)n << L.B;
    L.K = mass_factor(n, L.B, L.W);
    return true;
  }
  float wmax = 0.0f;
  for (u32 i = lane; i < n; i += 32) wmax = fmaxf(wmax, sane_weight(__ldg(w + i)));
#pragma unroll
  for (int o = 16; o; o >>= 1) wmax = fmaxf(wmax, __shfl_xor_sync(0xFFFFFFFFu, wmax, o));
  bool usable = wmax > 0.0f;
  if (usable) {
    L.B = bucket_bits(n);
    L.C = (u64)1 << L.B;
    L.sh = weight_shift(wmax, L.B);
    u64 acc = 0;
    for (u32 i = lane; i < n; i += 32) acc += quantise_bits(sane_weight(__ldg(w + i)), L.sh);
    L.W = warp_sum_u64(acc);
    L.nC = (u64)n << L.B;
    L.K = mass_factor(n, L.B, L.W);
    if (ck != nullptr) record_checkpoints(w, n, lane, L, ck);
  }
  if (lane == 0) {  // several warps may publish the same values at once: harmless
    *reinterpret_cast<volatile float*>(&memo->wmax) = usable ? wmax : 0.0f;
    *reinterpret_cast<volatile u64*>(&memo->W) = usable ? L.W : 0;
    __threadfence();
    *reinterpret_cast<volatile u32*>(&memo->stamp) = stamp;
  }
  return usable;
}

constexpr u32 kDirectEpt = 2, kDirectTile = 32 * kDirectEpt;
// masses of elements base + lane * kDirectEpt + k of the list (0 beyond its end); carryQ = quantised weight
// before `base`, advanced to the end of the tile
__device__ __forceinline__ void tile_masses(const float* __restrict__ w, u32 n, u32 base, u32 lane,
                                            const ListPrep& L, u64& carryQ, u64 (&m)[kDirectEpt]) {
  const u32 p0 = base + lane * kDirectEpt;
  u64 qs = 0;
#pragma unroll
  for (u32 k = 0; k < kDirectEpt; ++k) {
    m[k] = p0 + k < n ? quantise_bits(sane_weight(__ldg(w + p0 + k)), L.sh) : 0;
    qs += m[k];
  }
  u64 tq;
  u64 Q = carryQ + warp_excl_u64(qs, lane, tq);
  carryQ += tq;
  u64 g_prev = cum_mass(Q, L.W, L.nC, L.K);
#pragma unroll
  for (u32 k = 0; k < kDirectEpt; ++k) {
    if (p0 + k < n) {
      Q += m[k];
      const u64 g = cum_mass(Q, L.W, L.nC, L.K);
      m[k] = g - g_prev;
      g_prev = g;
    }
  }
}

// One full sweep of the list that stores (Q_b, D_b) at every chunk boundary b = k * kCkChunk, k >= 1.
__device__ void record_checkpoints(const float* __restrict__ w, u32 n, u32 lane, const ListPrep& L, Ckpt* ck) {
  u64 carryQ = 0, accD = 0;
  u64 m[kDirectEpt];
  for (u32 base = 0; base < n; base += kDirectTile) {
    if (base && base % kCkChunk == 0) {
      const u64 D = warp_sum_u64(accD);
      if (lane == 0) {
        volatile u64* dst = reinterpret_cast<volatile u64*>(ck + (base / kCkChunk - 1));
        dst[0] = carryQ;
        dst[1] = D;
      }
    }
    tile_masses(w, n, base, lane, L, carryQ, m);
#pragma unroll
    for (u32 k = 0; k < kDirectEpt; ++k)
      if (base + lane * kDirectEpt + k < n && m[k] < L.C) accD += L.C - m[k];
  }
}

// The sums at chunk boundary k (all zero at k = 0): quantised weight, deficit and excess before it.
__device__ __forceinline__ void ck_load(const Ckpt* ck, u32 k, const ListPrep& L, u64& Q, u64& D, u64& X) {
  Q = 0;
  D = 0;
  X = 0;
  if (k == 0 || ck == nullptr) return;
  const ulonglong2 e = __ldcg(reinterpret_cast<const ulonglong2*>(ck + (k - 1)));
  Q = e.x;
  D = e.y;
  X = D + cum_mass(Q, L.W, L.nC, L.K) - (((u64)k * kCkChunk) << L.B);
}

// (prob, alias) of slot p; every lane returns the same values.  ck: the vertex's checkpoints or
// nullptr.  v only labels error records.
__device__ Slot eval_slot(const float* __restrict__ w, u32 n, u32 p, u32 lane, const ListPrep& L,
                          const Ckpt* __restrict__ ck, u32 v, u32* err) {
  const u64 C = L.C;
  const u32 nck = ck ? (n - 1) / kCkChunk : 0;  // boundaries 1 .. nck carry checkpoints
  const u32 tp = p / kDirectTile, owner = (p % kDirectTile) / kDirectEpt;
  // sweep 1: masses from the boundary before p up to p; per-lane sums (on top of the boundary's) of
  // the deficits before p and of the excesses up to and including p
  const u32 kb = min(p / kCkChunk, nck);
  u64 baseQ, baseD, baseX;
  ck_load(ck, kb, L, baseQ, baseD, baseX);
  u64 carryQ = baseQ, accD = 0, accX = 0, Mp = 0;
  u64 saveQ = 0, saveD = 0, saveX = 0;  // the same sums at the start of p's tile
  u64 m[kDirectEpt];
  for (u32 t = kb * (kCkChunk / kDirectTile); t <= tp; ++t) {
    const u32 base = t * kDirectTile;
    if (t == tp) {
      saveQ = carryQ;
      saveD = accD;
      saveX = accX;
    }
    tile_masses(w, n, base, lane, L, carryQ, m);
#pragma unroll
    for (u32 k = 0; k < kDirectEpt; ++k) {
      const u32 idx = base + lane * kDirectEpt + k;
      if (idx < n && idx <= p) {
        if (idx == p) Mp = m[k];
        if (m[k] < C) accD += idx < p ? C - m[k] : 0;
        else accX += m[k] - C;
      }
    }
  }
  Mp = __shfl_sync(0xFFFFFFFFu, Mp, owner);
  Slot out;
  if (Mp < C) {
    // small: its donor is the first large whose running excess reaches the deficit before p
    const u64 T = baseD + warp_sum_u64(accD);
    out.prob = mass_to_prob_fast(Mp, L.B);
    out.alias = p;
    // The second sweep starts at the last chunk boundary whose excess is still below T (the donor lies
    // in that chunk) ...
    u64 cq, carryX, dummy;
    u32 start;
    {
      u32 lo = 0, hi = nck;
      while (lo < hi) {
        const u32 mid = (lo + hi + 1) >> 1;
        u64 q2, d2, x2;
        ck_load(ck, mid, L, q2, d2, x2);
        if (x2 < T) lo = mid;
        else hi = mid - 1;
      }
      ck_load(ck, lo, L, cq, dummy, carryX);
      start = lo * kCkChunk;
    }
    // ... or at p's tile, when the larges up to p do not reach T (the donor lies after p) and that is later
    if (baseX + warp_sum_u64(accX) < T && tp * kDirectTile > start) {
      start = tp * kDirectTile;
      cq = saveQ;
      carryX = baseX + warp_sum_u64(saveX);
    }
    bool found = false;
    for (u32 base = start; base < n && !found; base += kDirectTile) {
      tile_masses(w, n, base, lane, L, cq, m);
      u64 xs = 0;
#pragma unroll
      for (u32 k = 0; k < kDirectEpt; ++k)
        if (base + lane * kDirectEpt + k < n && m[k] >= C) xs += m[k] - C;
      u64 tx;
      u64 run = carryX + warp_excl_u64(xs, lane, tx);
      carryX += tx;
      u32 cand = kNoVertex;
#pragma unroll
      for (u32 k = 0; k < kDirectEpt; ++k) {
        const u32 idx = base + lane * kDirectEpt + k;
        if (idx < n && m[k] >= C) {
          run += m[k] - C;
          if (cand == kNoVertex && run >= T) cand = idx;
        }
      }
      const u32 hit = __ballot_sync(0xFFFFFFFFu, cand != kNoVertex);
      if (hit) {
        out.alias = __shfl_sync(0xFFFFFFFFu, cand, __ffs(hit) - 1);
        found = true;
      }
    }
    if (!found && lane == 0) dev_fail(err, DEV_ERR_INTERNAL, v, p, 11);
    return out;
  }
  // large: first small whose running deficit exceeds the excess up to and including p
  const u64 T = baseX + warp_sum_u64(accX);
  // the first large after p, from the tile already in registers and the tiles after it
  u32 next_large = kNoVertex;
  {
    u32 cand = kNoVertex;
#pragma unroll
    for (u32 k = 0; k < kDirectEpt; ++k) {
      const u32 idx = tp * kDirectTile + lane * kDirectEpt + k;
      if (idx < n && idx > p && m[k] >= C && cand == kNoVertex) cand = idx;
    }
    u32 hit = __ballot_sync(0xFFFFFFFFu, cand != kNoVertex);
    if (hit) next_large = __shfl_sync(0xFFFFFFFFu, cand, __ffs(hit) - 1);
    for (u32 base = (tp + 1) * kDirectTile; base < n && next_large == kNoVertex; base += kDirectTile) {
      tile_masses(w, n, base, lane, L, carryQ, m);
      cand = kNoVertex;
#pragma unroll
      for (u32 k = 0; k < kDirectEpt; ++k) {
        const u32 idx = base + lane * kDirectEpt + k;
        if (idx < n && m[k] >= C && cand == kNoVertex) cand = idx;
      }
      hit = __ballot_sync(0xFFFFFFFFu, cand != kNoVertex);
      if (hit) next_large = __shfl_sync(0xFFFFFFFFu, cand, __ffs(hit) - 1);
    }
  }
  out.prob = 1.0f;
  out.alias = p;
  if (next_large == kNoVertex) return out;  // the last large: no small can be left for it (D_total = X_total)
  // The second sweep starts at the last chunk boundary whose deficit does not exceed T (the crossing
  // lies in that chunk, or nowhere) ...
  u64 cq, carryD, dummy;
  u32 start;
  {
    u32 lo = 0, hi = nck;
    while (lo < hi) {
      const u32 mid = (lo + hi + 1) >> 1;
      u64 q2, d2, x2;
      ck_load(ck, mid, L, q2, d2, x2);
      if (d2 <= T) lo = mid;
      else hi = mid - 1;
    }
    ck_load(ck, lo, L, cq, carryD, dummy);
    start = lo * kCkChunk;
  }
  // ... or at p's tile, when the smalls before p do not exceed T (the crossing lies after p) and that is later
  if (baseD + warp_sum_u64(accD) <= T && tp * kDirectTile > start) {
    start = tp * kDirectTile;
    cq = saveQ;
    carryD = baseD + warp_sum_u64(saveD);
  }
  for (u32 base = start; base < n; base += kDirectTile) {
    tile_masses(w, n, base, lane, L, cq, m);
    u64 ds = 0;
#pragma unroll
    for (u32 k = 0; k < kDirectEpt; ++k)
      if (base + lane * kDirectEpt + k < n && m[k] < C) ds += C - m[k];
    u64 td;
    u64 run = carryD + warp_excl_u64(ds, lane, td);
    carryD += td;
    u64 at = 0;
    bool got = false;
#pragma unroll
    for (u32 k = 0; k < kDirectEpt; ++k) {
      if (base + lane * kDirectEpt + k < n && m[k] < C) {
        run += C - m[k];
        if (!got && run > T) {
          got = true;
          at = run;
        }
      }
    }
    const u32 hit = __ballot_sync(0xFFFFFFFFu, got);
    if (hit) {
      const u64 dsx = __shfl_sync(0xFFFFFFFFu, at, __ffs(hit) - 1);
      out.prob = mass_to_prob_fast(T + C - dsx, L.B);
      out.alias = next_large;
      return out;
    }
  }
  return out;  // every small was placed before this large: it owns one full bucket
}

// bool CheckConnect(src, dst) of the reference (include/gpu_graph.cuh:204-238) by the whole warp: the
// lanes probe 32 pivots of the sorted adjacency at once, so a list of d neighbours takes log_33(d)
// rounds of loads instead of the log_2(d) dependent loads of a lane searching alone.
__device__ __forceinline__ bool connected_warp(const u32* __restrict__ xadj, const u32* __restrict__ adjncy,
                                               u32 src, u32 dst, u32 lane) {
  u32 lo = __ldg(xadj + src), hi = __ldg(xadj + src + 1);  // dst, if present, lies in [lo, hi)
  while (hi - lo > 32) {
    const u32 span = hi - lo;
    const u32 x = __ldg(adjncy + lo + (u32)(((u64)(lane + 1) * span) / 33));  // 32 increasing pivots inside
    if (__ballot_sync(0xFFFFFFFFu, x == dst)) return true;
    const u32 c = __popc(__ballot_sync(0xFFFFFFFFu, x < dst));  // pivots below dst: a prefix of the lanes
    const u32 new_lo = c ? lo + (u32)(((u64)c * span) / 33) + 1 : lo;
    const u32 new_hi = c < 32 ? lo + (u32)(((u64)(c + 1) * span) / 33) : hi;
    lo = new_lo;
    hi = new_hi;
  }
  const bool hit = lo + lane < hi && __ldg(adjncy + lo + lane) == dst;
  return __ballot_sync(0xFFFFFFFFu, hit) != 0;
}

// One warp per walker, all steps in one launch.  Same draws and rules as walk_step.
template <int APP>
__global__ void __launch_bounds__(256, 4) walk_online_direct_kernel(const WalkArgs a, const float* __restrict__ wgt,
                                                                    PrepMemo* __restrict__ memo, u32 stamp,
                                                                    Ckpt* __restrict__ ck_all) {
  const u32 lane = threadIdx.x & 31;
  const u64 nwarps = ((u64)gridDim.x * blockDim.x) >> 5;
  u64 edges = 0;
  for (u64 w = ((u64)blockIdx.x * blockDim.x + threadIdx.x) >> 5; w < a.n; w += nwarps) {
    u32 cur = __ldg(a.starts + w), prev = kNoVertex, step = 0;
    u32* row = a.paths + w * a.hop_num;
    if (lane == 0) row[0] = cur;
    const u64 gw = a.walker_base + w * a.walker_stride;
    for (; step + 1 < a.hop_num; ++step) {
      Rand4 r = philox_tagged(a.seed, TAG_WALK, gw, step, 0);
      if (APP == SKW_APP_PPR && u01(r.z) < a.tp) break;
      if (cur >= a.V) {
        if (lane == 0) dev_fail(a.err, DEV_ERR_INDEX, cur, step, (u32)gw);
        break;
      }
      const u32 off = __ldg(a.xadj + cur);
      const u32 deg = __ldg(a.xadj + cur + 1) - off;
      if (deg == 0) break;
      const float* wl = wgt + off;
      ListPrep L;
      Ckpt* ck = (ck_all != nullptr && memo != nullptr && deg >= kCkMinDegree) ? ck_all + off / kCkChunk : nullptr;
      if (!list_prepare_memo(wl, deg, lane, L, memo ? memo + cur : nullptr, stamp, ck)) break;  // no usable weight
      u32 next;
      if (APP == SKW_APP_NODE2VEC && prev != kNoVertex) {
        for (u32 trial = 0;;) {
          const u32 col = __umulhi(r.x, deg);
          const Slot s = eval_slot(wl, deg, col, lane, L, ck, cur, a.err);
          const u32 cand = u01(r.y) < s.prob ? col : s.alias;
          next = __ldg(a.adjncy + (u64)off + cand);
          const float f = next == prev ? a.inv_p : (connected_warp(a.xadj, a.adjncy, prev, next, lane) ? 1.0f : a.inv_q);
          if (__fmul_rn(u01(r.w), a.fmax) < f) break;
          if (++trial == kN2vMaxTrials) break;  // keep the last proposal
          r = philox_tagged(a.seed, TAG_WALK, gw, step, trial);
        }
      } else {
        const u32 col = __umulhi(r.x, deg);
        const Slot s = eval_slot(wl, deg, col, lane, L, ck, cur, a.err);
        const u32 cand = u01(r.y) < s.prob ? col : s.alias;
        next = __ldg(a.adjncy + (u64)off + cand);
      }
      if (lane == 0) row[step + 1] = next;
      prev = cur;
      cur = next;
    }
    if (lane == 0) {
      a.lengths[w] = step;
      edges += step;
    }
  }
  add_edges(a.sum, edges);
}

int launch_walk_online_direct(skw_ctx* ctx, const WalkArgs& a, uint32_t app) {
  const u64 want = (a.n + 7) / 8;  // one warp per walker
  const int grid = (int)std::min<u64>(std::max<u64>(want, 1), (u64)ctx->sm_count * 32);
  cudaStream_t st = ctx->stream;
  // the per-vertex memo of (largest weight, total): allocated on first use when the graph has lists long
  // enough to use it, valid for one call (a new stamp per call; zero never names a call)
  PrepMemo* memo = nullptr;
  if (ctx->max_degree >= kMemoMinDegree) {
    if (!ctx->prep_memo) {
      SKW_CUDA(ctx, cudaMalloc(&ctx->prep_memo, sizeof(PrepMemo) * ((size_t)ctx->V + 1)));
      SKW_CUDA(ctx, cudaMemsetAsync(ctx->prep_memo, 0, sizeof(PrepMemo) * ((size_t)ctx->V + 1), st));
      ctx->prep_stamp = 0;
    }
    if (++ctx->prep_stamp == 0) {  // wrapped: forget every old entry
      SKW_CUDA(ctx, cudaMemsetAsync(ctx->prep_memo, 0, sizeof(PrepMemo) * ((size_t)ctx->V + 1), st));
      ctx->prep_stamp = 1;
    }
    memo = static_cast<PrepMemo*>(ctx->prep_memo);
  }
  Ckpt* ck_all = nullptr;
  if (memo != nullptr && ctx->max_degree >= kCkMinDegree) {
    if (!ctx->prep_ckpt) SKW_CUDA(ctx, cudaMalloc(&ctx->prep_ckpt, sizeof(Ckpt) * ((size_t)(ctx->E / kCkChunk) + 2)));
    ck_all = static_cast<Ckpt*>(ctx->prep_ckpt);  // validated by the memo's stamp: no clearing needed
  }
  const u32 stamp = ctx->prep_stamp;
  switch (app) {
    case SKW_APP_DEEPWALK: walk_online_direct_kernel<SKW_APP_DEEPWALK><<<grid, 256, 0, st>>>(a, ctx->adjwgt, memo, stamp, ck_all); break;
    case SKW_APP_PPR: walk_online_direct_kernel<SKW_APP_PPR><<<grid, 256, 0, st>>>(a, ctx->adjwgt, memo, stamp, ck_all); break;
    default: walk_online_direct_kernel<SKW_APP_NODE2VEC><<<grid, 256, 0, st>>>(a, ctx->adjwgt, memo, stamp, ck_all); break;
  }
  SKW_LAUNCHED(ctx);
  return SKW_OK;
}

}  // namespace skw
