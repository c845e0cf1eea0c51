// k-hop neighbour sampling, offline and online.
//
// Takes over OfflineSample / sample_kernel (src/offline_sample.cu:72-141, 443-513 of the
// reference) and OnlineGBSampleNew / sample_kernel (src/online_sample_new.cu:191-270, 459-547),
// writing the Jobs_result<NS> tree (include/sampler_result.cuh:226-260, 334-352, 421-426).
//
// The reference drains per-hop job queues with one thread (offline) or one warp (online) per
// frontier vertex.  Here a hop is one launch with one thread per OUTPUT cell: thread
// (seed s, parent idx, child j) reads the parent vertex, makes its own Philox draw keyed by
// (seed id, child cell, hop) and stores one coalesced word; no queues and no atomics on the data
// path.  Online mode first builds the tables of the distinct vertices of the hop's frontier with
// the degree-bucketed builders, then runs the same draw kernel.
#include <algorithm>
#include <string>

#include <cub/device/device_scan.cuh>

#include "skw_ctx.h"

namespace skw {

int frontier_collect(skw_ctx* ctx, const u32* verts, u64 units, u32 width, u32 cells, u32 offs,
                     const u32* alive_lengths, bool new_round);

struct KhopArgs {
  const u32* xadj;
  const u32* adjncy;
  const Slot* slots;
  u32* data;
  u32* lens;
  unsigned long long* sum;
  u32* err;
  u64 n;
  u64 seed;
  u64 instance_base;
  u64 instance_stride;
  u32 V;
  u32 cells, lens_per;
  u32 offs_parent, offs_child, width_parent, fanout, hop, flags;
};

__global__ void __launch_bounds__(256) khop_init_kernel(const u32* __restrict__ seeds, u64 n,
                                                        u32 cells, u32* __restrict__ data) {
  for (u64 s = (u64)blockIdx.x * blockDim.x + threadIdx.x; s < n; s += (u64)gridDim.x * blockDim.x)
    data[s * cells] = seeds[s];
}

__global__ void __launch_bounds__(256) khop_hop_kernel(const KhopArgs a) {
  const u64 per_seed = (u64)a.width_parent * a.fanout;
  const u64 total = a.n * per_seed;
  u64 got_sum = 0;
  for (u64 u = (u64)blockIdx.x * blockDim.x + threadIdx.x; u < total; u += (u64)gridDim.x * blockDim.x) {
    const u64 s = u / per_seed;
    const u32 rem = (u32)(u - s * per_seed);
    const u32 idx = rem / a.fanout, j = rem - idx * a.fanout;
    u32* row = a.data + s * a.cells;
    const u32 v = row[a.offs_parent + idx];
    u32 out = SKW_INVALID_VERTEX, got = 0;
    if (v != SKW_INVALID_VERTEX) {
      if (v >= a.V) {
        dev_fail(a.err, DEV_ERR_INDEX, v, idx, a.hop);
      } else {
        const u32 off = __ldg(a.xadj + v), deg = __ldg(a.xadj + v + 1) - off;
        if (deg) {
          if ((a.flags & SKW_KHOP_TAKE_ALL) && a.fanout >= deg) {
            got = deg;
            if (j < deg) out = __ldg(a.adjncy + (u64)off + j);
          } else {
            const Rand4 r = philox_tagged(a.seed, TAG_KHOP, a.instance_base + s * a.instance_stride, rem, a.hop);
            const u32 col = __umulhi(r.x, deg);
            if (a.flags & SKW_KHOP_UNBIASED) {
              out = ldg_once(a.adjncy + (u64)off + col);
              got = a.fanout;
              goto store;
            }
            const Slot sl = load_slot(a.slots + (u64)off + col);
            if (!(sl.prob < 0.0f)) {
              const u32 cand = u01(r.y) < sl.prob ? col : sl.alias;
              if (cand >= deg) {  // a table that does not belong to this graph
                dev_fail(a.err, DEV_ERR_INDEX, v, cand, 23);
              } else {
                out = ldg_once(a.adjncy + (u64)off + cand);
                got = a.fanout;
              }
            }
          }
        }
      }
    }
  store:
    row[a.offs_child + rem] = out;
    if (j == 0) {
      a.lens[s * a.lens_per + a.offs_parent + idx] = got;
      got_sum += got;
    }
  }
#pragma unroll
  for (int o = 16; o; o >>= 1) got_sum += __shfl_xor_sync(0xFFFFFFFFu, got_sum, o);
  if ((threadIdx.x & 31) == 0 && got_sum) atomicAdd(a.sum, (unsigned long long)got_sum);
}

// SKW_KHOP_DISTINCT: one warp per parent vertex.  A parent whose degree is <= the fan-out hands over
// every neighbour once.  Otherwise trial t (t = lane + 32 * round, 11 rounds at most, as the reference's
// roll_atomic, src/online_sample_new.cu:73-111) draws a column with its own Philox words, keyed by
// (seed id, parent index, trial, hop); a draw counts when its column was not drawn by an earlier trial.
// "Earlier" is decided without atomics: columns accepted in earlier rounds sit in a per-warp list in
// shared memory, and inside a round the lowest lane holding a column wins (match_any), so the result
// is the one a sequential pass over the trials gives.
constexpr u32 kDistinctMaxFanout = 256, kDistinctRounds = 11;
__global__ void __launch_bounds__(256) khop_distinct_kernel(const KhopArgs a) {
  __shared__ u32 s_seen[8][kDistinctMaxFanout];
  const u32 lane = threadIdx.x & 31, wib = threadIdx.x >> 5;
  const u64 warp = ((u64)blockIdx.x * blockDim.x + threadIdx.x) >> 5;
  const u64 nwarps = ((u64)gridDim.x * blockDim.x) >> 5;
  const u64 parents = a.n * a.width_parent;
  const u32 f = a.fanout;
  u32* seen = s_seen[wib];
  u64 got_sum = 0;
  for (u64 u = warp; u < parents; u += nwarps) {
    const u64 s = u / a.width_parent;
    const u32 idx = (u32)(u - s * a.width_parent);
    u32* row = a.data + s * a.cells;
    u32* child = row + a.offs_child + (u64)idx * f;
    const u32 v = row[a.offs_parent + idx];
    u32 got = 0;
    u32 off = 0, deg = 0;
    if (v != SKW_INVALID_VERTEX) {
      if (v >= a.V) {
        if (lane == 0) dev_fail(a.err, DEV_ERR_INDEX, v, idx, a.hop);
      } else {
        off = __ldg(a.xadj + v);
        deg = __ldg(a.xadj + v + 1) - off;
      }
    }
    if (deg && f >= deg) {
      for (u32 j = lane; j < deg; j += 32) child[j] = __ldg(a.adjncy + (u64)off + j);
      got = deg;
    } else if (deg) {
      const u64 gi = a.instance_base + s * a.instance_stride;
      for (u32 round = 0; round < kDistinctRounds && got < f; ++round) {
        const u32 t = round * 32 + lane;
        const Rand4 r = philox_tagged(a.seed, TAG_KHOP, gi, idx, (t << 8) | 0x80u | a.hop);
        const u32 col = __umulhi(r.x, deg);
        const Slot sl = load_slot(a.slots + (u64)off + col);
        if (sl.prob < 0.0f) break;  // vertex without usable weight: the same in every lane
        u32 cand = u01(r.y) < sl.prob ? col : sl.alias;
        if (cand >= deg) {  // a table that does not belong to this graph
          dev_fail(a.err, DEV_ERR_INDEX, v, cand, 24);
          cand = 0;
        }
        bool fresh = true;
        for (u32 i = 0; i < got; ++i) fresh = fresh && seen[i] != cand;
        const u32 same = __match_any_sync(0xFFFFFFFFu, cand);
        fresh = fresh && lane == (u32)(__ffs(same) - 1);
        const u32 acc = __ballot_sync(0xFFFFFFFFu, fresh);
        const u32 at = got + __popc(acc & ((1u << lane) - 1u));
        if (fresh && at < f) {
          seen[at] = cand;
          child[at] = ldg_once(a.adjncy + (u64)off + cand);
        }
        got = min(f, got + (u32)__popc(acc));
        __syncwarp();
      }
    }
    for (u32 j = got + lane; j < f; j += 32) child[j] = SKW_INVALID_VERTEX;
    if (lane == 0) {
      a.lens[s * a.lens_per + a.offs_parent + idx] = got;
      got_sum += got;
    }
    __syncwarp();  // the list is reused by the next parent
  }
  if (lane == 0 && got_sum) atomicAdd(a.sum, (unsigned long long)got_sum);
}

static int khop_check(skw_ctx* ctx, const skw_khop_params* prm) {
  if (prm->nhops < 1 || prm->nhops > 4) return fail(ctx, SKW_ERR_ARG, "skw_sample_khop: nhops must be 1..4");
  if (prm->mode > SKW_MODE_ONLINE) return fail(ctx, SKW_ERR_ARG, "skw_sample_khop: unknown mode %u", prm->mode);
  u64 w = 1, cells = 1;
  for (u32 h = 0; h < prm->nhops; ++h) {
    if (prm->fanout[h] == 0) return fail(ctx, SKW_ERR_ARG, "skw_sample_khop: fan-out of hop %u is 0", h + 1);
    if ((prm->flags & SKW_KHOP_DISTINCT) && !(prm->flags & SKW_KHOP_UNBIASED) && prm->fanout[h] > kDistinctMaxFanout)
      return fail(ctx, SKW_ERR_ARG, "skw_sample_khop: SKW_KHOP_DISTINCT takes fan-outs up to %u, hop %u asks for %u",
                  kDistinctMaxFanout, h + 1, prm->fanout[h]);
    w *= prm->fanout[h];
    cells += w;
    if (cells > 0x7FFFFFFFull) return fail(ctx, SKW_ERR_ARG, "skw_sample_khop: tree of %llu cells per seed is too large",
                                            (unsigned long long)cells);
  }
  return SKW_OK;
}

}  // namespace skw

using namespace skw;

extern "C" {

int skw_khop_layout(const skw_khop_params* prm, uint32_t* cells_per_seed, uint32_t* lengths_per_seed) {
  if (!prm) return SKW_ERR_ARG;
  int rc = khop_check(nullptr, prm);
  if (rc != SKW_OK) return rc;
  uint32_t w = 1, cells = 0, lens = 0;
  for (uint32_t h = 0; h <= prm->nhops; ++h) {
    if (h) w *= prm->fanout[h - 1];
    if (h == prm->nhops) lens = cells;
    cells += w;
  }
  if (cells_per_seed) *cells_per_seed = cells;
  if (lengths_per_seed) *lengths_per_seed = lens;
  return SKW_OK;
}

// Argument and state checks of the k-hop entry points.
static int khop_validate(skw_ctx* ctx, const skw_khop_params* prm) {
  int rc = khop_check(ctx, prm);
  if (rc != SKW_OK) return rc;
  if (!ctx->xadj) return fail(ctx, SKW_ERR_STATE, "skw_sample_khop: no graph resident");
  const bool unbiased = (prm->flags & SKW_KHOP_UNBIASED) != 0;
  const bool online = prm->mode == SKW_MODE_ONLINE && !unbiased;
  if (!online && !unbiased && !ctx->table_ready)
    return fail(ctx, SKW_ERR_STATE, "skw_sample_khop: offline mode needs skw_alias_build_offline or skw_alias_import first");
  if (online && !ctx->adjwgt) return fail(ctx, SKW_ERR_STATE, "skw_sample_khop: online mode needs the edge weights");
  return SKW_OK;
}

// Packed result tree: the cells of a seed's row that hold a sample, in row order (the seed, its hop-1
// samples, the hop-2 samples of the first of them, of the second ...), seeds back to back.  One warp
// per seed: count the cells of the row that are not SKW_INVALID_VERTEX ...
__global__ void __launch_bounds__(256) khop_count_cells_kernel(const u32* __restrict__ data, u64 n, u32 cells,
                                                               u64* __restrict__ count) {
  const u32 lane = threadIdx.x & 31;
  const u64 nwarps = ((u64)gridDim.x * blockDim.x) >> 5;
  for (u64 s = ((u64)blockIdx.x * blockDim.x + threadIdx.x) >> 5; s < n; s += nwarps) {
    const u32* row = data + s * cells;
    u32 c = 0;
    for (u32 x = lane; x < cells; x += 32) c += ldg_once(row + x) != SKW_INVALID_VERTEX ? 1u : 0u;
#pragma unroll
    for (int o = 16; o; o >>= 1) c += __shfl_xor_sync(0xFFFFFFFFu, c, o);
    if (lane == 0) count[s] = c;
  }
}

// ... and, once the counts are prefix-summed into offs, copy them out in order.  Cells that do not
// fit the capacity are left out; *total tells the host what the batch needs.
__global__ void __launch_bounds__(256) khop_pack_kernel(const u32* __restrict__ data, u64 n, u32 cells,
                                                        const u64* __restrict__ offs, u32* __restrict__ packed,
                                                        u64 capacity, u64* __restrict__ total) {
  const u32 lane = threadIdx.x & 31, below = (1u << lane) - 1u;
  const u64 nwarps = ((u64)gridDim.x * blockDim.x) >> 5;
  for (u64 s = ((u64)blockIdx.x * blockDim.x + threadIdx.x) >> 5; s < n; s += nwarps) {
    const u32* row = data + s * cells;
    u64 o = __ldg(offs + s);
    for (u32 x0 = 0; x0 < cells; x0 += 32) {
      const u32 x = x0 + lane;
      const u32 v = x < cells ? ldg_once(row + x) : SKW_INVALID_VERTEX;
      const u32 have = __ballot_sync(0xFFFFFFFFu, v != SKW_INVALID_VERTEX);
      const u64 at = o + __popc(have & below);
      if (v != SKW_INVALID_VERTEX && at < capacity) packed[at] = v;
      o += __popc(have);
    }
    if (s == n - 1 && lane == 0) *total = o;
  }
}

// Queue the kernels of one batch of seeds on the context's stream (sampled edges add up in d_sum[0]).
static int khop_launch(skw_ctx* ctx, const skw_khop_params* prm, const uint32_t* d_seeds, uint64_t n,
                       uint32_t* d_data, uint32_t* d_sample_lengths, uint64_t instance_base,
                       bool first_of_call) {
  const bool unbiased = (prm->flags & SKW_KHOP_UNBIASED) != 0;
  const bool online = prm->mode == SKW_MODE_ONLINE && !unbiased;
  int rc;
  if (online) {
    drop_records(ctx);  // online builds overwrite table slots
    if ((rc = alloc_table(ctx)) != SKW_OK) return rc;
  }
  if (!n) return SKW_OK;
  uint32_t width[6], offs[6], cells = 0, w = 1;
  for (uint32_t h = 0; h <= prm->nhops; ++h) {
    if (h) w *= prm->fanout[h - 1];
    width[h] = w;
    offs[h] = cells;
    cells += w;
  }
  KhopArgs a;
  a.xadj = ctx->xadj;
  a.adjncy = ctx->adjncy;
  a.slots = ctx->slots;
  a.data = d_data;
  a.lens = d_sample_lengths;
  a.sum = reinterpret_cast<unsigned long long*>(ctx->d_sum);
  a.err = ctx->d_err;
  a.n = n;
  a.seed = prm->seed;
  a.instance_base = instance_base;
  a.instance_stride = prm->instance_stride ? prm->instance_stride : 1;
  a.V = ctx->V;
  a.cells = cells;
  a.lens_per = offs[prm->nhops];
  a.flags = prm->flags;
  cudaStream_t st = ctx->stream;
  const uint64_t cap = (uint64_t)ctx->sm_count * 16;
  uint64_t want = (n + 255) / 256;
  khop_init_kernel<<<(int)(want < cap ? want : cap), 256, 0, st>>>(d_seeds, n, cells, d_data);
  SKW_LAUNCHED(ctx);
  for (uint32_t h = 0; h < prm->nhops; ++h) {
    // A table built earlier in this call (an earlier hop, an earlier slice of the seeds) stays good:
    // only the first collection of a call opens a new round of claims, every later one skips the
    // vertices that already hold one.
    if (online && (rc = frontier_collect(ctx, d_data, n * width[h], width[h], cells, offs[h], nullptr,
                                         first_of_call && h == 0)) != SKW_OK)
      return rc;
    a.offs_parent = offs[h];
    a.offs_child = offs[h + 1];
    a.width_parent = width[h];
    a.fanout = prm->fanout[h];
    a.hop = h + 1;
    if ((prm->flags & SKW_KHOP_DISTINCT) && !unbiased) {
      want = (n * width[h] + 7) / 8;  // one warp per parent vertex
      khop_distinct_kernel<<<(int)(want < cap ? want : cap), 256, 0, st>>>(a);
    } else {
      want = (n * width[h + 1] + 255) / 256;
      khop_hop_kernel<<<(int)(want < cap ? want : cap), 256, 0, st>>>(a);
    }
    SKW_LAUNCHED(ctx);
  }
  return SKW_OK;
}

int skw_sample_khop_device(skw_ctx* ctx, const skw_khop_params* prm, const uint32_t* d_seeds,
                           uint64_t n, uint32_t* d_data, uint32_t* d_sample_lengths, float* ms,
                           uint64_t* sampled_edges) {
  if (!ctx || !prm) return SKW_ERR_ARG;
  if (n && (!d_seeds || !d_data || !d_sample_lengths)) return fail(ctx, SKW_ERR_ARG, "skw_sample_khop: null buffer");
  int rc = khop_validate(ctx, prm);
  if (rc != SKW_OK) return rc;
  DeviceGuard g(ctx->device);
  cudaStream_t st = ctx->stream;
  if ((rc = err_reset(ctx)) != SKW_OK) return rc;
  SKW_CUDA(ctx, cudaMemsetAsync(ctx->d_sum, 0, sizeof(uint64_t), st));
  SKW_CUDA(ctx, cudaEventRecord(ctx->ev0, st));
  if ((rc = khop_launch(ctx, prm, d_seeds, n, d_data, d_sample_lengths, prm->instance_base, true)) != SKW_OK) return rc;
  SKW_CUDA(ctx, cudaEventRecord(ctx->ev1, st));
  SKW_CUDA(ctx, cudaMemcpyAsync(ctx->h_sum, ctx->d_sum, sizeof(uint64_t), cudaMemcpyDeviceToHost, st));
  if ((rc = err_check(ctx, "skw_sample_khop")) != SKW_OK) return rc;
  if (ms) SKW_CUDA(ctx, cudaEventElapsedTime(ms, ctx->ev0, ctx->ev1));
  if (sampled_edges) *sampled_edges = *ctx->h_sum;
  return SKW_OK;
}

int skw_sample_khop(skw_ctx* ctx, const skw_khop_params* prm, const uint32_t* h_seeds, uint64_t n,
                    uint32_t* h_data, uint32_t* h_sample_lengths, float* ms, uint64_t* sampled_edges) {
  if (!ctx || !prm) return SKW_ERR_ARG;
  uint32_t cells = 0, lens = 0;
  int rc = skw_khop_layout(prm, &cells, &lens);
  if (rc != SKW_OK) return fail(ctx, rc, "skw_sample_khop: bad hop description");
  if (n && (!h_seeds || !h_data || !h_sample_lengths)) return fail(ctx, SKW_ERR_ARG, "skw_sample_khop: null buffer");
  if ((rc = khop_validate(ctx, prm)) != SKW_OK) return rc;
  DeviceGuard g(ctx->device);
  const size_t nb = sizeof(uint32_t) * (size_t)n;
  if ((rc = ensure_bytes(ctx, &ctx->stage[0], &ctx->stage_bytes[0], nb)) != SKW_OK) return rc;
  if ((rc = ensure_bytes(ctx, &ctx->stage[1], &ctx->stage_bytes[1], nb * cells)) != SKW_OK) return rc;
  if ((rc = ensure_bytes(ctx, &ctx->stage[2], &ctx->stage_bytes[2], nb * lens)) != SKW_OK) return rc;
  uint32_t* d_seeds = static_cast<uint32_t*>(ctx->stage[0]);
  uint32_t* d_data = static_cast<uint32_t*>(ctx->stage[1]);
  uint32_t* d_lens = static_cast<uint32_t*>(ctx->stage[2]);
  cudaStream_t st = ctx->stream, side = ctx->side_stream;
  // A result tree is dense (every cell crosses the bus), so a large batch runs as two or four slices
  // of seeds: while the kernels of slice c run on the context's stream, the tree of slice c - 1 goes
  // home on the side stream.  Seed ids, hence samples, do not depend on the slicing, and in online mode
  // a vertex whose table an earlier slice built is not built again.  What a slice still costs is the
  // per-hop launch sequence over a smaller frontier (measured on B200, online 2-hop 25 x 10 with 65,536
  // seeds: 2.52 ms per call unsliced, 2.29 ms in two slices, 2.45 ms in four), so slices stay large.
  const uint32_t slices = n >= (1u << 19) ? 4 : (n >= (1u << 16) ? 2 : 1);
  const uint64_t per = (n + slices - 1) / slices;
  const uint64_t stride = prm->instance_stride ? prm->instance_stride : 1;
  if ((rc = err_reset(ctx)) != SKW_OK) return rc;
  SKW_CUDA(ctx, cudaMemsetAsync(ctx->d_sum, 0, sizeof(uint64_t), st));
  if (n) SKW_CUDA(ctx, cudaMemcpyAsync(d_seeds, h_seeds, nb, cudaMemcpyHostToDevice, st));
  SKW_CUDA(ctx, cudaEventRecord(ctx->ev0, st));
  for (uint32_t c = 0; c < slices; ++c) {
    const uint64_t base = (uint64_t)c * per;
    if (base >= n) break;
    const uint64_t nc = std::min<uint64_t>(per, n - base);
    rc = khop_launch(ctx, prm, d_seeds + base, nc, d_data + base * cells, d_lens + base * lens,
                     prm->instance_base + base * stride, c == 0);
    if (rc != SKW_OK) {
      cudaStreamSynchronize(side);
      cudaStreamSynchronize(st);
      return rc;
    }
    SKW_CUDA(ctx, cudaEventRecord(ctx->pk_ready[c], st));
    SKW_CUDA(ctx, cudaStreamWaitEvent(side, ctx->pk_ready[c], 0));
    SKW_CUDA(ctx, cudaMemcpyAsync(h_data + base * cells, d_data + base * cells, sizeof(uint32_t) * (size_t)nc * cells,
                                  cudaMemcpyDeviceToHost, side));
    SKW_CUDA(ctx, cudaMemcpyAsync(h_sample_lengths + base * lens, d_lens + base * lens,
                                  sizeof(uint32_t) * (size_t)nc * lens, cudaMemcpyDeviceToHost, side));
  }
  SKW_CUDA(ctx, cudaEventRecord(ctx->ev1, st));
  SKW_CUDA(ctx, cudaMemcpyAsync(ctx->h_sum, ctx->d_sum, sizeof(uint64_t), cudaMemcpyDeviceToHost, st));
  const int rc_side = cudaStreamSynchronize(side) == cudaSuccess ? SKW_OK : SKW_ERR_CUDA;
  if ((rc = err_check(ctx, "skw_sample_khop")) != SKW_OK) return rc;
  if (rc_side != SKW_OK) return fail(ctx, SKW_ERR_CUDA, "skw_sample_khop: copying the result failed");
  if (ms) SKW_CUDA(ctx, cudaEventElapsedTime(ms, ctx->ev0, ctx->ev1));
  if (sampled_edges) *sampled_edges = *ctx->h_sum;
  return SKW_OK;
}

// Host buffers, packed result tree (see khop_pack_kernel): only cells that hold a sample cross the
// bus.  Slices as in skw_sample_khop; per slice the kernels, the count of each row's samples, their
// prefix sum and the packing are queued for all slices before the host waits for anything, the size of
// a slice's packed part comes back through a pinned word and its copy starts as soon as that is known.
int skw_sample_khop_packed(skw_ctx* ctx, const skw_khop_params* prm, const uint32_t* h_seeds, uint64_t n,
                           uint32_t* h_packed, uint64_t capacity_cells, uint32_t* h_sample_lengths,
                           uint64_t* cells_out, float* ms, uint64_t* sampled_edges) {
  if (!ctx || !prm) return SKW_ERR_ARG;
  if (!cells_out) return fail(ctx, SKW_ERR_ARG, "skw_sample_khop_packed: cells must not be null");
  *cells_out = 0;
  if (ms) *ms = 0;
  if (sampled_edges) *sampled_edges = 0;
  uint32_t cells = 0, lens = 0;
  int rc = skw_khop_layout(prm, &cells, &lens);
  if (rc != SKW_OK) return fail(ctx, rc, "skw_sample_khop_packed: bad hop description");
  if (n && (!h_seeds || !h_sample_lengths)) return fail(ctx, SKW_ERR_ARG, "skw_sample_khop_packed: null buffer");
  if ((rc = khop_validate(ctx, prm)) != SKW_OK) return rc;
  if (!n) return SKW_OK;
  DeviceGuard g(ctx->device);
  cudaStream_t st = ctx->stream, side = ctx->side_stream;
  const uint32_t slices = n >= (1u << 19) ? 4 : (n >= (1u << 16) ? 2 : 1);
  const uint64_t per = (n + slices - 1) / slices;
  const uint64_t stride = prm->instance_stride ? prm->instance_stride : 1;
  const size_t nb = sizeof(uint32_t) * (size_t)n;
  const size_t offs_bytes = (sizeof(u64) * (size_t)per * 2 + 255) & ~(size_t)255;  // counts, then offsets
  size_t tmp_bytes = 0;
  SKW_CUDA(ctx, cub::DeviceScan::ExclusiveSum(nullptr, tmp_bytes, (const u64*)nullptr, (u64*)nullptr, (long long)per, st));
  if ((rc = ensure_bytes(ctx, &ctx->stage[0], &ctx->stage_bytes[0], nb)) != SKW_OK) return rc;
  if ((rc = ensure_bytes(ctx, &ctx->stage[1], &ctx->stage_bytes[1], nb * cells)) != SKW_OK) return rc;
  if ((rc = ensure_bytes(ctx, &ctx->stage[2], &ctx->stage_bytes[2], nb * lens)) != SKW_OK) return rc;
  if ((rc = ensure_bytes(ctx, &ctx->stage[3], &ctx->stage_bytes[3], offs_bytes + tmp_bytes)) != SKW_OK) return rc;
  uint32_t* d_seeds = static_cast<uint32_t*>(ctx->stage[0]);
  uint32_t* d_data = static_cast<uint32_t*>(ctx->stage[1]);
  uint32_t* d_lens = static_cast<uint32_t*>(ctx->stage[2]);
  u64* d_cnt = static_cast<u64*>(ctx->stage[3]);
  u64* d_offs = d_cnt + per;
  void* d_tmp = reinterpret_cast<char*>(ctx->stage[3]) + offs_bytes;
  // one packing buffer per slice, kept at its high-water size; first guess: every cell of the tree
  uint64_t cap[4] = {}, nc_of[4] = {};
  for (uint32_t c = 0; c < slices; ++c) {
    const uint64_t base = (uint64_t)c * per;
    if (base >= n) break;
    nc_of[c] = std::min<uint64_t>(per, n - base);
    const uint64_t full = nc_of[c] * cells;
    uint64_t guess = full;
    if (ctx->stage[4 + c] && ctx->stage_bytes[4 + c] >= sizeof(u32) * 1024) guess = ctx->stage_bytes[4 + c] / sizeof(u32);
    if ((rc = ensure_bytes(ctx, &ctx->stage[4 + c], &ctx->stage_bytes[4 + c], sizeof(u32) * (size_t)guess)) != SKW_OK) return rc;
    cap[c] = std::min<uint64_t>(ctx->stage_bytes[4 + c] / sizeof(u32), full);
  }
  if ((rc = err_reset(ctx)) != SKW_OK) return rc;
  const uint64_t grid_cap = (uint64_t)ctx->sm_count * 16;
  auto count_and_pack = [&](uint32_t c, bool recount) -> int {
    const uint64_t base = (uint64_t)c * per, nc = nc_of[c];
    const uint64_t want = (nc + 7) / 8;  // one warp per seed
    const int grid = (int)(want < grid_cap ? want : grid_cap);
    if (recount) {
      khop_count_cells_kernel<<<grid, 256, 0, st>>>(d_data + base * cells, nc, cells, d_cnt);
      SKW_LAUNCHED(ctx);
      size_t tb = tmp_bytes;
      SKW_CUDA(ctx, cub::DeviceScan::ExclusiveSum(d_tmp, tb, d_cnt, d_offs, (long long)nc, st));
      SKW_LAUNCHED(ctx);
    }
    khop_pack_kernel<<<grid, 256, 0, st>>>(d_data + base * cells, nc, cells, d_offs,
                                           static_cast<u32*>(ctx->stage[4 + c]), cap[c], ctx->d_tot + c);
    SKW_LAUNCHED(ctx);
    SKW_CUDA(ctx, cudaEventRecord(ctx->pk_ready[c], st));
    SKW_CUDA(ctx, cudaStreamWaitEvent(side, ctx->pk_ready[c], 0));
    SKW_CUDA(ctx, cudaMemcpyAsync(ctx->h_tot + c, ctx->d_tot + c, sizeof(u64), cudaMemcpyDeviceToHost, side));
    SKW_CUDA(ctx, cudaEventRecord(ctx->pk_tot[c], side));
    return SKW_OK;
  };
  auto body = [&]() -> int {
    SKW_CUDA(ctx, cudaMemsetAsync(ctx->d_sum, 0, sizeof(uint64_t), st));
    SKW_CUDA(ctx, cudaMemcpyAsync(d_seeds, h_seeds, nb, cudaMemcpyHostToDevice, st));
    SKW_CUDA(ctx, cudaEventRecord(ctx->ev0, st));
    for (uint32_t c = 0; c < slices && nc_of[c]; ++c) {
      const uint64_t base = (uint64_t)c * per, nc = nc_of[c];
      int r = khop_launch(ctx, prm, d_seeds + base, nc, d_data + base * cells, d_lens + base * lens,
                          prm->instance_base + base * stride, c == 0);
      if (r != SKW_OK) return r;
      if (c + 1 == slices || !nc_of[c + 1]) SKW_CUDA(ctx, cudaEventRecord(ctx->ev1, st));
      if ((r = count_and_pack(c, true)) != SKW_OK) return r;
      SKW_CUDA(ctx, cudaMemcpyAsync(h_sample_lengths + base * lens, d_lens + base * lens,
                                    sizeof(uint32_t) * (size_t)nc * lens, cudaMemcpyDeviceToHost, side));
    }
    uint64_t total_cells = 0;
    bool fits = h_packed != nullptr;
    for (uint32_t c = 0; c < slices && nc_of[c]; ++c) {
      SKW_CUDA(ctx, cudaEventSynchronize(ctx->pk_tot[c]));
      uint64_t slice_cells = ctx->h_tot[c];
      if (fits && total_cells + slice_cells > capacity_cells) fits = false;  // keep going: the caller gets the size
      if (fits && slice_cells > cap[c]) {
        // the slice outgrew its packing buffer: grow it and pack again.  The offsets of this slice are
        // gone once a later slice was counted, so they are computed again unless it is the last one.
        int r = ensure_bytes(ctx, &ctx->stage[4 + c], &ctx->stage_bytes[4 + c], sizeof(u32) * (size_t)(nc_of[c] * cells));
        if (r != SKW_OK) return r;
        cap[c] = nc_of[c] * cells;
        if ((r = count_and_pack(c, true)) != SKW_OK) return r;
        SKW_CUDA(ctx, cudaEventSynchronize(ctx->pk_tot[c]));
        slice_cells = ctx->h_tot[c];
      }
      if (fits) {
        SKW_CUDA(ctx, cudaStreamWaitEvent(ctx->copy_stream, ctx->pk_ready[c], 0));
        SKW_CUDA(ctx, cudaMemcpyAsync(h_packed + total_cells, ctx->stage[4 + c], sizeof(u32) * (size_t)slice_cells,
                                      cudaMemcpyDeviceToHost, ctx->copy_stream));
      }
      total_cells += slice_cells;
    }
    SKW_CUDA(ctx, cudaMemcpyAsync(ctx->h_sum, ctx->d_sum, sizeof(uint64_t), cudaMemcpyDeviceToHost, st));
    SKW_CUDA(ctx, cudaStreamSynchronize(side));
    SKW_CUDA(ctx, cudaStreamSynchronize(ctx->copy_stream));
    int r = err_check(ctx, "skw_sample_khop_packed");  // synchronises the context's stream
    if (r != SKW_OK) return r;
    *cells_out = total_cells;
    if (ms) SKW_CUDA(ctx, cudaEventElapsedTime(ms, ctx->ev0, ctx->ev1));
    if (sampled_edges) *sampled_edges = *ctx->h_sum;
    if (!fits)
      return fail(ctx, SKW_ERR_ARG, "skw_sample_khop_packed: the result needs %llu cells, the buffer holds %llu",
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

}  // extern "C"
