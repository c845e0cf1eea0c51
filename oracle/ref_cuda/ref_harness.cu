// Harness around the reference's OWN offline walk (wpybtw/Skywalker, src/offline_walk.cu:181-230:
// OfflineWalk -> sample_kernel_static, lines 75-124) and its OWN offline 2-hop sampler
// (src/offline_sample.cu:443-513: OfflineSample -> sample_kernel, lines 72-141) and its OWN unbiased
// walk (src/unbiased_walk.cu:194-278: UnbiasedWalk -> UnbiasedWalkKernelStatic, lines 104-130),
// compiled from the reference sources where they lie.  TEST / MEASUREMENT INFRASTRUCTURE ONLY: nothing in the shipped
// library links this.
//
// Only these three entry functions of the reference are driven, because their kernels are bounded:
// the walks are per-thread loops of hop_num - 1 iterations, the sampler drains job queues whose
// sizes are fixed by the seed count and the fan-outs (every pop is one atomic, there is no wait on
// another thread), and every index is derived from xadj / the table.  The
// reference's table constructors (include/alias_table_new.cuh:637-708 spins in `while (alive)`) and
// its online kernels (src/online_walk.cu:94-165, persistent without a grid barrier) are never
// launched: the alias table is handed in by the caller as the reference's own three arrays
// (gpu_graph::prob_array, alias_array, valid; include/gpu_graph.cuh:40-60).
//
// The kernel draws its column as floor(curand_uniform * degree); curand_uniform lies in (0, 1], so
// the column can equal the degree (src/offline_walk.cu:100-108) and the reads then land one entry
// past the vertex's list.  Every array is therefore allocated with spare entries after its end, and
// the spare table entries are {prob 1, alias 0}, the spare neighbour is vertex 0.
#include <cstdint>
#include <cstring>
#include <vector>

#include "app.cuh"

// flags the compiled reference files read; their definitions live in src/main.cu, which is not built
DEFINE_bool(v, false, "verbose");
DEFINE_bool(debug, false, "debug");
DEFINE_bool(printresult, false, "printresult");
DEFINE_bool(static, true, "using static scheduling");
DEFINE_bool(buffer, false, "buffered write for memory");
DEFINE_bool(umgraph, false, "");
DEFINE_bool(gmgraph, true, "");
DEFINE_bool(hmgraph, false, "");
DEFINE_int32(gmid, 0, "");
DEFINE_bool(ol, false, "");
DEFINE_bool(randomweight, false, "");
DEFINE_bool(pf, false, "");
DEFINE_bool(ab, false, "");
DEFINE_double(pfr, 1.0, "");
DEFINE_bool(umresult, false, "");
DEFINE_bool(umtable, false, "");
DEFINE_bool(hmtable, false, "");
DEFINE_bool(umbuf, false, "");
DEFINE_bool(node2vec, false, "");
DEFINE_bool(peritr, false, "");
DEFINE_bool(itl, true, "");
DEFINE_bool(replica, false, "");
DEFINE_bool(loc, false, "");
DEFINE_double(p, 2.0, "");
DEFINE_double(q, 0.5, "");
DEFINE_double(tp, 0.0, "");
DEFINE_double(hd, 1.0, "");
DEFINE_int32(m, 4, "");
DEFINE_int32(device, 0, "");
DEFINE_int32(weightrange, 2, "");
DEFINE_string(input, "", "");

namespace {
const size_t kSpare = 64;
struct Dev {
  void* p = nullptr;
  ~Dev() { cudaFree(p); }
  template <typename T>
  T* alloc(size_t n) {
    return cudaMalloc(&p, sizeof(T) * n) == cudaSuccess ? static_cast<T*>(p) : nullptr;
  }
};
}  // namespace

// Runs `repeats` launches of the reference walk over the same walkers and returns the best wall time
// the reference itself reports (OfflineWalk's return value: seconds around its kernel launch).
// paths is n x hop_num (row per walker, the reference's Jobs_result<RW> layout), lengths has n entries.
// Returns 0, or a negative value when an argument or a CUDA call fails.
extern "C" int skwref_offline_walk(int device, uint32_t V, uint64_t E, const uint32_t* h_xadj,
                                   const uint32_t* h_adjncy, const float* h_prob, const uint32_t* h_alias,
                                   const unsigned char* h_valid, const uint32_t* h_starts, uint32_t n,
                                   uint32_t hop_num, int repeats, uint32_t* h_paths, uint32_t* h_lengths,
                                   double* best_seconds) {
  if (!h_xadj || !h_adjncy || !h_prob || !h_alias || !h_valid || !h_starts || !h_paths || !h_lengths || !n ||
      hop_num < 2 || E > 0xFFFFFF00ull)
    return -1;
  // every index the kernel forms must stay inside the padded arrays: check the inputs on the host
  if (h_xadj[0] != 0 || h_xadj[V] != E) return -1;
  for (uint32_t v = 0; v < V; ++v)
    if (h_xadj[v] > h_xadj[v + 1]) return -1;
  for (uint64_t e = 0; e < E; ++e)
    if (h_adjncy[e] >= V) return -1;
  for (uint32_t v = 0; v < V; ++v)
    for (uint32_t i = h_xadj[v]; i < h_xadj[v + 1]; ++i)
      if (h_alias[i] >= h_xadj[v + 1] - h_xadj[v]) return -1;
  for (uint32_t i = 0; i < n; ++i)
    if (h_starts[i] >= V) return -1;
  if (cudaSetDevice(device) != cudaSuccess) return -2;
  FLAGS_static = true;
  FLAGS_buffer = false;
  Dev dx, da, dp, dl, dv, dd, dal, dlen;
  uint32_t* xadj = dx.alloc<uint32_t>((size_t)V + 1 + kSpare);
  uint32_t* adjncy = da.alloc<uint32_t>(E + kSpare);
  float* prob = dp.alloc<float>(E + kSpare);
  uint32_t* alias = dl.alloc<uint32_t>(E + kSpare);
  char* valid = dv.alloc<char>((size_t)V + kSpare);
  uint32_t* data = dd.alloc<uint32_t>((size_t)n * hop_num);
  char* alive = dal.alloc<char>(n);
  uint32_t* length = dlen.alloc<uint32_t>(n);
  if (!xadj || !adjncy || !prob || !alias || !valid || !data || !alive || !length) return -2;
  std::vector<float> ones(kSpare, 1.0f);
  bool ok = cudaMemcpy(xadj, h_xadj, sizeof(uint32_t) * ((size_t)V + 1), cudaMemcpyHostToDevice) == cudaSuccess &&
            cudaMemcpy(adjncy, h_adjncy, sizeof(uint32_t) * E, cudaMemcpyHostToDevice) == cudaSuccess &&
            cudaMemset(adjncy + E, 0, sizeof(uint32_t) * kSpare) == cudaSuccess &&
            cudaMemcpy(prob, h_prob, sizeof(float) * E, cudaMemcpyHostToDevice) == cudaSuccess &&
            cudaMemcpy(prob + E, ones.data(), sizeof(float) * kSpare, cudaMemcpyHostToDevice) == cudaSuccess &&
            cudaMemcpy(alias, h_alias, sizeof(uint32_t) * E, cudaMemcpyHostToDevice) == cudaSuccess &&
            cudaMemset(alias + E, 0, sizeof(uint32_t) * kSpare) == cudaSuccess &&
            cudaMemcpy(valid, h_valid, V, cudaMemcpyHostToDevice) == cudaSuccess;
  if (!ok) return -2;
  gpu_graph g;
  g.adjncy = adjncy;
  g.adjwgt = nullptr;
  g.xadj = xadj;
  g.degree_list = nullptr;
  g.outDegree = nullptr;
  g.prob_array = prob;
  g.alias_array = alias;
  g.valid = valid;
  g.vtx_num = V;
  g.edge_num = (edge_t)E;
  g.avg_degree = V ? (edge_t)(E / V) : 0;
  g.MaxDegree = 0;
  g.device_id = device;
  g.result = nullptr;
  g.local_vtx_offset = 0;
  g.local_edge_offset = 0;
  g.local_vtx_num = V;
  g.local_edge_num = (uint)E;
  Walker walker(g, device);
  walker.num_seed = n;
  walker.prob_array = prob;
  walker.alias_array = alias;
  walker.valid = valid;
  std::memset(&walker.result, 0, sizeof(walker.result));
  walker.result.size = n;
  walker.result.hop_num = hop_num;
  walker.result.data = data;
  walker.result.alive = alive;
  walker.result.length = length;
  walker.result.device_id = device;
  std::vector<uint32_t> rows((size_t)n * hop_num, 0xFFFFFFFFu);
  for (uint32_t i = 0; i < n; ++i) rows[(size_t)i * hop_num] = h_starts[i];
  double best = 1e30;
  for (int r = 0; r < (repeats > 0 ? repeats : 1); ++r) {
    if (cudaMemcpy(data, rows.data(), sizeof(uint32_t) * rows.size(), cudaMemcpyHostToDevice) != cudaSuccess ||
        cudaMemset(alive, 1, n) != cudaSuccess || cudaMemset(length, 0, sizeof(uint32_t) * n) != cudaSuccess)
      return -2;
    const double t = OfflineWalk(walker);
    if (cudaDeviceSynchronize() != cudaSuccess) return -3;
    if (t < best) best = t;
  }
  if (cudaMemcpy(h_paths, data, sizeof(uint32_t) * rows.size(), cudaMemcpyDeviceToHost) != cudaSuccess ||
      cudaMemcpy(h_lengths, length, sizeof(uint32_t) * n, cudaMemcpyDeviceToHost) != cudaSuccess)
    return -2;
  if (best_seconds) *best_seconds = best;
  return 0;
}


// The reference's offline 2-hop neighbour sampling over the same kind of inputs: seeds, fan-outs
// {1, f1, f2} (its hop_num = 3, the depth its job frontier is compiled for), the caller's alias table.
// data is n x (1 + f1 + f1 * f2) (seed, hop-1 samples, hop-2 samples of each of them: the reference's
// Jobs_result<NS> layout, cells without a sample keep what its initSeed2 kernel wrote),
// sample_lengths is n x (1 + f1).  Returns 0, or a negative value when an argument or a CUDA call fails.
extern "C" int skwref_offline_sample(int device, uint32_t V, uint64_t E, const uint32_t* h_xadj,
                                     const uint32_t* h_adjncy, const float* h_prob, const uint32_t* h_alias,
                                     const unsigned char* h_valid, const uint32_t* h_seeds, uint32_t n,
                                     uint32_t f1, uint32_t f2, int blocks_per_sm, int repeats, uint32_t* h_data,
                                     uint32_t* h_sample_lengths, double* best_seconds,
                                     unsigned long long* sampled_edges) {
  if (!h_xadj || !h_adjncy || !h_prob || !h_alias || !h_valid || !h_seeds || !h_data || !h_sample_lengths || !n ||
      !f1 || !f2 || f1 > 64 || f2 > 64 || (uint64_t)n * f1 * f2 > (1ull << 26) || E > 0xFFFFFF00ull)
    return -1;
  if (h_xadj[0] != 0 || h_xadj[V] != E) return -1;
  for (uint32_t v = 0; v < V; ++v)
    if (h_xadj[v] > h_xadj[v + 1]) return -1;
  for (uint64_t e = 0; e < E; ++e)
    if (h_adjncy[e] >= V) return -1;
  for (uint32_t v = 0; v < V; ++v)
    for (uint32_t i = h_xadj[v]; i < h_xadj[v + 1]; ++i)
      if (h_alias[i] >= h_xadj[v + 1] - h_xadj[v]) return -1;
  for (uint32_t i = 0; i < n; ++i)
    if (h_seeds[i] >= V) return -1;
  if (device != 0 || cudaSetDevice(device) != cudaSuccess) return -2;  // Jobs_result::init picks device 0 itself
  FLAGS_peritr = false;  // the one-launch kernel over job queues
  FLAGS_buffer = false;
  FLAGS_umresult = false;
  FLAGS_hd = 1.0;
  FLAGS_m = blocks_per_sm > 0 ? blocks_per_sm : 4;  // the reference's default is 4 thread blocks per SM
  Dev dx, da, dp, dl, dv;
  uint32_t* xadj = dx.alloc<uint32_t>((size_t)V + 1 + kSpare);
  uint32_t* adjncy = da.alloc<uint32_t>(E + kSpare);
  float* prob = dp.alloc<float>(E + kSpare);
  uint32_t* alias = dl.alloc<uint32_t>(E + kSpare);
  char* valid = dv.alloc<char>((size_t)V + kSpare);
  if (!xadj || !adjncy || !prob || !alias || !valid) return -2;
  std::vector<float> ones(kSpare, 1.0f);
  bool ok = cudaMemcpy(xadj, h_xadj, sizeof(uint32_t) * ((size_t)V + 1), cudaMemcpyHostToDevice) == cudaSuccess &&
            cudaMemcpy(adjncy, h_adjncy, sizeof(uint32_t) * E, cudaMemcpyHostToDevice) == cudaSuccess &&
            cudaMemset(adjncy + E, 0, sizeof(uint32_t) * kSpare) == cudaSuccess &&
            cudaMemcpy(prob, h_prob, sizeof(float) * E, cudaMemcpyHostToDevice) == cudaSuccess &&
            cudaMemcpy(prob + E, ones.data(), sizeof(float) * kSpare, cudaMemcpyHostToDevice) == cudaSuccess &&
            cudaMemcpy(alias, h_alias, sizeof(uint32_t) * E, cudaMemcpyHostToDevice) == cudaSuccess &&
            cudaMemset(alias + E, 0, sizeof(uint32_t) * kSpare) == cudaSuccess &&
            cudaMemcpy(valid, h_valid, V, cudaMemcpyHostToDevice) == cudaSuccess;
  if (!ok) return -2;
  gpu_graph g;
  g.adjncy = adjncy;
  g.adjwgt = nullptr;
  g.xadj = xadj;
  g.degree_list = nullptr;
  g.outDegree = nullptr;
  g.prob_array = prob;
  g.alias_array = alias;
  g.valid = valid;
  g.vtx_num = V;
  g.edge_num = (edge_t)E;
  g.avg_degree = V ? (edge_t)(E / V) : 0;
  g.MaxDegree = 0;
  g.device_id = device;
  g.result = nullptr;
  g.local_vtx_offset = 0;
  g.local_edge_offset = 0;
  g.local_vtx_num = V;
  g.local_edge_num = (uint)E;
  uint hops[3] = {1, f1, f2};
  std::vector<uint32_t> seeds(h_seeds, h_seeds + n);
  double best = 1e30;
  unsigned long long edges = 0;
  const size_t cells = 1 + (size_t)f1 + (size_t)f1 * f2, lens = 1 + (size_t)f1;
  for (int r = 0; r < (repeats > 0 ? repeats : 1); ++r) {
    Sampler_new sampler(g, device);
    sampler.num_seed = n;
    sampler.prob_array = prob;
    sampler.alias_array = alias;
    sampler.valid = valid;
    // Jobs_result<NS> neither initialises nor allocates these two, and its Free() hands them to cudaFree
    sampler.result.alive = nullptr;
    sampler.result.length = nullptr;
    sampler.result.init(n, 3, hops, seeds.data(), device, V);  // allocates data, lengths and the job queues
    if (sampler.result.length_per_sample != cells || sampler.result.size_of_sample_lengths != lens) return -4;
    // The kernel's queue of the next hop is filled while other thread blocks already drain it, and
    // SampleFrontier::Add publishes a slot (atomicAdd on the size) before it writes the job into it
    // (include/frontier.cuh:236-246), so a slot can be read before it is written.  Cleared slots read
    // as "no job" (val = false) or, half written, as vertex 0 / sample 0 / offset 0: every index the
    // kernel forms from them stays inside the arrays, whatever the interleaving.  (Jobs read too early
    // are dropped by the reference: its hop-2 result is incomplete, hop 1 is not affected.)
    for (int i = 1; i < 3; ++i)
      if (cudaMemset(sampler.result.frontier.data[i], 0,
                     sizeof(sampleJob<uint>) * (size_t)sampler.result.frontier.capacity[i]) != cudaSuccess)
        return -2;
    const double t = OfflineSample(sampler);
    if (cudaDeviceSynchronize() != cudaSuccess) return -3;
    if (t < best) best = t;
    edges = sampler.sampled_edges;
    const bool last = r + 1 >= (repeats > 0 ? repeats : 1);
    if (last && (cudaMemcpy(h_data, sampler.result.data, sizeof(uint32_t) * n * cells, cudaMemcpyDeviceToHost) !=
                     cudaSuccess ||
                 cudaMemcpy(h_sample_lengths, sampler.result.sample_lengths, sizeof(uint32_t) * n * lens,
                            cudaMemcpyDeviceToHost) != cudaSuccess))
      return -2;
    sampler.prob_array = nullptr;  // the table belongs to this function, not to the sampler
    sampler.alias_array = nullptr;
    sampler.valid = nullptr;
    sampler.Free(true);  // data, job counters, the per-hop overflow queues
    // what init() allocates and Free() leaves behind
    cudaFree(sampler.result.sample_lengths);
    cudaFree(sampler.result.hops);
    cudaFree(sampler.result.offsets);
    cudaFree(sampler.result.seeds);
    for (int i = 0; i < 3; ++i) cudaFree(sampler.result.frontier.data[i]);
    cudaFree(sampler.result.frontier.sizes);
    cudaFree(sampler.result.frontier.floor);
    delete[] sampler.result.hops_h;
    delete[] sampler.result.high_degrees_h;
  }
  if (best_seconds) *best_seconds = best;
  if (sampled_edges) *sampled_edges = edges;
  return 0;
}


// The reference's unbiased walk with its stop rule (every step ends the walk with probability tp, or
// at a vertex without out-edges; the neighbour is floor(curand_uniform * degree), no table), one
// thread per walker.  lengths has n entries; h_paths (n x hop_num) may be null when only the lengths
// are wanted.  Returns 0, or a negative value when an argument or a CUDA call fails.
extern "C" int skwref_unbiased_walk(int device, uint32_t V, uint64_t E, const uint32_t* h_xadj,
                                    const uint32_t* h_adjncy, const uint32_t* h_starts, uint32_t n,
                                    uint32_t hop_num, double tp, int repeats, uint32_t* h_paths,
                                    uint32_t* h_lengths, double* best_seconds) {
  if (!h_xadj || !h_adjncy || !h_starts || !h_lengths || !n || hop_num < 2 || E > 0xFFFFFF00ull || tp < 0.0 ||
      tp >= 1.0)
    return -1;
  if (h_xadj[0] != 0 || h_xadj[V] != E) return -1;
  for (uint32_t v = 0; v < V; ++v)
    if (h_xadj[v] > h_xadj[v + 1]) return -1;
  for (uint64_t e = 0; e < E; ++e)
    if (h_adjncy[e] >= V) return -1;
  for (uint32_t i = 0; i < n; ++i)
    if (h_starts[i] >= V) return -1;
  if (cudaSetDevice(device) != cudaSuccess) return -2;
  FLAGS_static = true;  // UnbiasedWalkKernelStatic: a bounded loop per thread
  FLAGS_buffer = false;
  FLAGS_peritr = false;
  FLAGS_node2vec = false;
  FLAGS_tp = tp;
  Dev dx, da, dd, dal, dlen, dst;
  uint32_t* xadj = dx.alloc<uint32_t>((size_t)V + 1 + kSpare);
  uint32_t* adjncy = da.alloc<uint32_t>(E + kSpare);  // the column can equal the degree: one entry past a list
  uint32_t* data = dd.alloc<uint32_t>((size_t)n * hop_num);
  char* alive = dal.alloc<char>(n);
  uint32_t* length = dlen.alloc<uint32_t>(n);
  uint32_t* starts = dst.alloc<uint32_t>(n);
  if (!xadj || !adjncy || !data || !alive || !length || !starts) return -2;
  bool ok = cudaMemcpy(xadj, h_xadj, sizeof(uint32_t) * ((size_t)V + 1), cudaMemcpyHostToDevice) == cudaSuccess &&
            cudaMemcpy(adjncy, h_adjncy, sizeof(uint32_t) * E, cudaMemcpyHostToDevice) == cudaSuccess &&
            cudaMemset(adjncy + E, 0, sizeof(uint32_t) * kSpare) == cudaSuccess &&
            cudaMemcpy(starts, h_starts, sizeof(uint32_t) * n, cudaMemcpyHostToDevice) == cudaSuccess;
  if (!ok) return -2;
  gpu_graph g;
  g.adjncy = adjncy;
  g.adjwgt = nullptr;
  g.xadj = xadj;
  g.degree_list = nullptr;
  g.outDegree = nullptr;
  g.prob_array = nullptr;
  g.alias_array = nullptr;
  g.valid = nullptr;
  g.vtx_num = V;
  g.edge_num = (edge_t)E;
  g.avg_degree = V ? (edge_t)(E / V) : 0;
  g.MaxDegree = 0;
  g.device_id = device;
  g.result = nullptr;
  g.local_vtx_offset = 0;
  g.local_edge_offset = 0;
  g.local_vtx_num = V;
  g.local_edge_num = (uint)E;
  Walker walker(g, device);
  walker.num_seed = n;
  walker.prob_array = nullptr;
  walker.alias_array = nullptr;
  walker.valid = nullptr;
  std::memset(&walker.result, 0, sizeof(walker.result));
  walker.result.size = n;
  walker.result.hop_num = hop_num;
  walker.result.data = data;
  walker.result.alive = alive;
  walker.result.length = length;
  walker.result.device_id = device;
  double best = 1e30;
  for (int r = 0; r < (repeats > 0 ? repeats : 1); ++r) {
    // rows of 0xFFFFFFFF with the start vertex in column 0 (a strided copy of the start array)
    if (cudaMemset(data, 0xFF, sizeof(uint32_t) * (size_t)n * hop_num) != cudaSuccess ||
        cudaMemcpy2D(data, sizeof(uint32_t) * hop_num, starts, sizeof(uint32_t), sizeof(uint32_t), n,
                     cudaMemcpyDeviceToDevice) != cudaSuccess ||
        cudaMemset(alive, 1, n) != cudaSuccess || cudaMemset(length, 0, sizeof(uint32_t) * n) != cudaSuccess)
      return -2;
    const double t = UnbiasedWalk(walker);
    if (cudaDeviceSynchronize() != cudaSuccess) return -3;
    if (t < best) best = t;
  }
  if ((h_paths && cudaMemcpy(h_paths, data, sizeof(uint32_t) * (size_t)n * hop_num, cudaMemcpyDeviceToHost) !=
                      cudaSuccess) ||
      cudaMemcpy(h_lengths, length, sizeof(uint32_t) * n, cudaMemcpyDeviceToHost) != cudaSuccess)
    return -2;
  if (best_seconds) *best_seconds = best;
  return 0;
}
