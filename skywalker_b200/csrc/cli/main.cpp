// skywalker -- command-line driver with the reference's flag surface.
//
// Takes over src/main.cu of the reference: same flag names and defaults (main.cu:32-109, plus
// --weight from src/api/bias_static.cu:8), same presets (main.cu:156-184), one host thread per GPU
// (main.cu:252-270), same stdout rows (main.cu:398-420: optional table-build ms row, time ms row,
// MSEPS row; --csv prints one line).  Everything it computes goes through the C ABI of
// include/skywalker_b200.h.  Flags of the reference's out-of-core memory placements
// (--umgraph, --hmgraph, --umtable, --hmtable, --umresult, --umbuf, --pf, --ab, --pfr) are
// accepted and ignored: graph and tables always live in HBM (the reference's --gmgraph).
//
// Additions: --seed (Philox seed, default 42), --randstart (uniformly random start vertices
// instead of the reference's "walker i starts at vertex i"), --rmat_scale / --rmat_ef (seeded
// synthetic graph instead of --input), --records (fused walk records), --batches (k-hop batches),
// --d is honoured when given explicitly together with --deepwalk / --ppr / --node2vec (the
// reference overrides it with 100).
#include <algorithm>
#include <chrono>
#include <cstdint>
#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <map>
#include <string>
#include <thread>
#include <vector>

#include <cuda_runtime.h>
#ifdef SKW_HAVE_NCCL
#include <nccl.h>
#endif

#include "skywalker_b200.h"
#include "rendezvous.h"

namespace {

struct Flag {
  enum Kind { BOOL, INT, DOUBLE, STRING } kind;
  std::string value;
  bool set = false;
};
std::map<std::string, Flag> g_flags;

void def(const char* name, Flag::Kind k, const char* dflt) { g_flags[name] = Flag{k, dflt, false}; }
bool fb(const char* n) { return g_flags.at(n).value == "true" || g_flags.at(n).value == "1"; }
long fi(const char* n) { return atol(g_flags.at(n).value.c_str()); }
double fd(const char* n) { return atof(g_flags.at(n).value.c_str()); }
const std::string& fs(const char* n) { return g_flags.at(n).value; }
bool was_set(const char* n) { return g_flags.at(n).set; }
void setb(const char* n, bool v) { g_flags.at(n).value = v ? "true" : "false"; }
void seti(const char* n, long v) { g_flags.at(n).value = std::to_string(v); }

// gflags command-line conventions: --name=value, --name value, -name, --boolname, --noboolname
int parse_flags(int argc, char** argv) {
  for (int i = 1; i < argc; ++i) {
    std::string a = argv[i];
    if (a.size() < 2 || a[0] != '-') {
      fprintf(stderr, "unexpected argument '%s'\n", a.c_str());
      return 1;
    }
    a = a.substr(a[1] == '-' ? 2 : 1);
    std::string name = a, val;
    bool has_val = false;
    const size_t eq = a.find('=');
    if (eq != std::string::npos) {
      name = a.substr(0, eq);
      val = a.substr(eq + 1);
      has_val = true;
    }
    auto it = g_flags.find(name);
    if (it == g_flags.end() && name.rfind("no", 0) == 0) {
      auto it2 = g_flags.find(name.substr(2));
      if (it2 != g_flags.end() && it2->second.kind == Flag::BOOL && !has_val) {
        it2->second.value = "false";
        it2->second.set = true;
        continue;
      }
    }
    if (it == g_flags.end()) {
      fprintf(stderr, "ERROR: unknown command line flag '%s'\n", name.c_str());
      return 1;
    }
    Flag& f = it->second;
    if (f.kind == Flag::BOOL) {
      if (!has_val) val = "true";
      if (val == "1" || val == "t" || val == "true" || val == "yes" || val == "y") val = "true";
      else if (val == "0" || val == "f" || val == "false" || val == "no" || val == "n") val = "false";
      else {
        fprintf(stderr, "ERROR: illegal value '%s' for boolean flag '%s'\n", val.c_str(), name.c_str());
        return 1;
      }
    } else if (!has_val) {
      if (i + 1 >= argc) {
        fprintf(stderr, "ERROR: flag '%s' is missing its argument\n", name.c_str());
        return 1;
      }
      val = argv[++i];
    }
    f.value = val;
    f.set = true;
  }
  return 0;
}

void define_flags() {
  def("input", Flag::STRING, "");
  def("ngpu", Flag::INT, "1");
  def("s", Flag::BOOL, "true");
  def("n", Flag::INT, "4000");
  def("k", Flag::INT, "2");
  def("d", Flag::INT, "2");
  def("hd", Flag::DOUBLE, "1");
  def("ol", Flag::BOOL, "false");
  def("rw", Flag::BOOL, "false");
  def("dw", Flag::BOOL, "false");
  def("randomweight", Flag::BOOL, "false");
  def("weightrange", Flag::INT, "2");
  def("sage", Flag::BOOL, "false");
  def("deepwalk", Flag::BOOL, "false");
  def("node2vec", Flag::BOOL, "false");
  def("ppr", Flag::BOOL, "false");
  def("p", Flag::DOUBLE, "2.0");
  def("q", Flag::DOUBLE, "0.5");
  def("tp", Flag::DOUBLE, "0.0");
  def("hmtable", Flag::BOOL, "false");
  def("dt", Flag::BOOL, "true");
  def("umgraph", Flag::BOOL, "true");
  def("hmgraph", Flag::BOOL, "false");
  def("gmgraph", Flag::BOOL, "false");
  def("gmid", Flag::INT, "1");
  def("umtable", Flag::BOOL, "false");
  def("umresult", Flag::BOOL, "false");
  def("umbuf", Flag::BOOL, "false");
  def("cache", Flag::BOOL, "false");
  def("debug", Flag::BOOL, "false");
  def("bias", Flag::BOOL, "true");
  def("full", Flag::BOOL, "false");
  def("stream", Flag::BOOL, "false");
  def("v", Flag::BOOL, "false");
  def("printresult", Flag::BOOL, "false");
  def("edgecut", Flag::BOOL, "true");
  def("itl", Flag::BOOL, "true");
  def("twc", Flag::BOOL, "false");
  def("static", Flag::BOOL, "true");
  def("buffer", Flag::BOOL, "false");
  def("m", Flag::INT, "4");
  def("peritr", Flag::BOOL, "false");
  def("sp", Flag::BOOL, "false");
  def("pf", Flag::BOOL, "true");
  def("ab", Flag::BOOL, "true");
  def("pfr", Flag::DOUBLE, "1.0");
  def("async", Flag::BOOL, "false");
  def("replica", Flag::BOOL, "false");
  def("built", Flag::BOOL, "false");
  def("gmem", Flag::BOOL, "false");
  def("newsampler", Flag::BOOL, "true");
  def("csv", Flag::BOOL, "false");
  def("weight", Flag::BOOL, "true");
  // additions
  def("seed", Flag::INT, "42");
  def("randstart", Flag::BOOL, "false");
  def("rmat_scale", Flag::INT, "0");
  def("rmat_ef", Flag::INT, "16");
  def("records", Flag::BOOL, "false");
  def("batches", Flag::INT, "1");
  def("gather", Flag::BOOL, "true");
  def("replacement", Flag::BOOL, "false");
}

#define LOGV(...)                      \
  do {                                 \
    if (fb("v")) {                     \
      printf("%s:%d HOST: ", "main.cpp", __LINE__); \
      printf(__VA_ARGS__);             \
    }                                  \
  } while (0)

struct DevResult {
  float table_ms = 0, time_s = 0;
  uint64_t sampled = 0;
  int rc = 0;
  std::string err;
};

struct Shared {
  Rendezvous rv;
  int ndev;
  uint32_t V = 0;
  uint64_t E = 0;
  long n_total;
  int depth;
  std::vector<uint32_t> hops;
#ifdef SKW_HAVE_NCCL
  std::vector<ncclComm_t> comms;
#endif
  std::vector<uint32_t> gathered_lengths;  // rank 0 fills it when --gather
  std::vector<uint32_t> gathered_paths;    // and the path rows, device by device
  int gather_rows = 0;                     // GPU 0's decision whether the rows fit beside its own data
};

int fail_dev(DevResult& r, skw_ctx* ctx, int rc, const char* what) {
  r.rc = rc;
  r.err = std::string(what) + ": " + (ctx ? skw_last_error(ctx) : skw_last_global_error());
  return rc;
}

int run_device(int dev, Shared& sh, DevResult& out) {
  skw_ctx* ctx = nullptr;
  int rc = skw_ctx_create(dev, &ctx);
  if (rc) return fail_dev(out, nullptr, rc, "skw_ctx_create");
  struct Guard {
    skw_ctx* c;
    ~Guard() { skw_ctx_destroy(c); }
  } guard{ctx};
  const bool bias = fb("bias");
  // graph: replicated in this GPU's HBM
  if (fi("rmat_scale") > 0) {
    rc = skw_graph_generate_rmat(ctx, (uint32_t)fi("rmat_scale"), 0, (uint64_t)fi("rmat_ef") << fi("rmat_scale"), 0.57,
                                 0.19, 0.19, 0, 1, 7);
  } else {
    int mode = 0;
    if (!bias || !fb("weight")) mode = 1;
    if (fb("dw")) mode = 2;
    if (fb("randomweight")) mode = 3;
    rc = skw_graph_load_gr(ctx, fs("input").c_str(), mode, (uint32_t)fi("weightrange"), 0);
  }
  if (rc) return fail_dev(out, ctx, rc, "graph");
  uint32_t V, maxdeg;
  uint64_t E;
  skw_graph_info(ctx, &V, &E, &maxdeg);
  if (dev == 0) {
    sh.V = V;
    sh.E = E;
  }
  LOGV("device %d: %u nodes, %llu edges, max degree %u\n", dev, V, (unsigned long long)E, maxdeg);
  const bool online = fb("ol");
  if (bias && !online) {
    float ms = 0;
    bool sliced = false;
#ifdef SKW_HAVE_NCCL
    // More than one GPU: the slot array is cut into ndev * kPieces equal chunks of S slots; GPU d builds
    // the vertices that overlap chunks d, ndev + d, 2 ndev + d ... (a vertex straddling a boundary is
    // built by both neighbours, with identical bits), and piece k -- the ndev neighbouring chunks
    // k * ndev .. k * ndev + ndev - 1 -- is all-gathered in place over NCCL while the GPUs already build
    // their chunk of piece k + 1; one all-reduce of the per-vertex flags completes every GPU's table
    // (the reference assembles edge-balanced slices through pinned host memory,
    // include/sampler.cuh:151-158, include/gpu_graph.cuh:282-291).  --dt=0 (one shared host table)
    // has no meaning here.
    if (sh.ndev > 1 && !sh.comms.empty() && E > 0) {
      constexpr int kPieces = 4;
      const int parts = sh.ndev * kPieces;
      std::vector<uint32_t> xadj((size_t)V + 1);
      rc = skw_graph_download(ctx, xadj.data(), nullptr, nullptr);
      if (rc) return fail_dev(out, ctx, rc, "skw_graph_download");  // the others learn of it in agree() below
      const uint64_t S = (E + parts - 1) / parts;
      std::vector<uint32_t> vb(parts), ve(parts);
      for (int r = 0; r < parts; ++r) {
        const uint64_t lo = std::min<uint64_t>((uint64_t)r * S, E), hi = std::min<uint64_t>((uint64_t)(r + 1) * S, E);
        if (hi > lo) {
          vb[r] = (uint32_t)(std::upper_bound(xadj.begin(), xadj.end(), (uint32_t)lo) - xadj.begin()) - 1;
          ve[r] = (uint32_t)(std::upper_bound(xadj.begin(), xadj.end(), (uint32_t)(hi - 1)) - xadj.begin());
        } else {
          vb[r] = ve[r] = V;
        }
      }
      vb[0] = 0;
      ve[parts - 1] = V;
      for (int r = 0; r + 1 < parts; ++r) {  // vertices without edges between two chunks
        ve[r] = std::max(ve[r], std::min(vb[r + 1], V));
        if (vb[r] > ve[r]) vb[r] = ve[r];
      }
      cudaStream_t st;
      cudaStreamCreate(&st);
      {  // the first collective of a communicator pays its connection set-up: keep that out of the table time
        uint32_t* d_one = nullptr;
        cudaMalloc(&d_one, sizeof(uint32_t));
        cudaMemsetAsync(d_one, 0, sizeof(uint32_t), st);
        ncclAllReduce(d_one, d_one, 1, ncclUint32, ncclSum, sh.comms[dev], st);
        cudaStreamSynchronize(st);
        cudaFree(d_one);
      }
      const auto t0 = std::chrono::steady_clock::now();
      float build_ms = 0;
      uint64_t* slots = nullptr;
      uint8_t* valid = nullptr;
      for (int k = 0; k < kPieces; ++k) {
        const int c = k * sh.ndev + dev;
        float piece_ms = 0;
        rc = skw_alias_build_offline(ctx, vb[c], ve[c], &piece_ms);  // returns when the chunk is built
        build_ms += piece_ms;
        if (!sh.rv.agree(rc == 0)) {  // nobody enters a collective that another device will not join
          cudaStreamSynchronize(st);
          cudaStreamDestroy(st);
          if (rc) return fail_dev(out, ctx, rc, "skw_alias_build_offline (slice)");
          out.rc = SKW_ERR_STATE;
          out.err = "another device failed before the table all-gather";
          return out.rc;
        }
        if (!slots) {
          const void* slots_c = nullptr;
          const uint8_t* valid_c = nullptr;
          skw_alias_device_ptrs(ctx, &slots_c, &valid_c);
          slots = (uint64_t*)slots_c;  // 8-byte {prob, alias} slots, 1024 spare entries past E
          valid = (uint8_t*)valid_c;
        }
        ncclAllGather(slots + (size_t)c * S, slots + (size_t)k * sh.ndev * S, S, ncclUint64, sh.comms[dev], st);
      }
      ncclAllReduce(valid, valid, V, ncclUint8, ncclMax, sh.comms[dev], st);  // set by the builders, zero elsewhere
      cudaStreamSynchronize(st);
      const float wall_ms = std::chrono::duration<float, std::milli>(std::chrono::steady_clock::now() - t0).count();
      LOGV("device %d: %d chunks built in %.2f ms of kernel time, table complete after %.2f ms (pieces all-gathered "
           "over NCCL beside the builds)\n", dev, kPieces, build_ms, wall_ms);
      ms = wall_ms;
      cudaStreamDestroy(st);
      sliced = true;
    }
#endif
    if (!sliced) {
      rc = skw_alias_build_offline(ctx, 0, V, &ms);
      if (rc) return fail_dev(out, ctx, rc, "skw_alias_build_offline");
    }
    out.table_ms = ms;
    if (fb("records") && fb("rw") && !fb("node2vec")) {
      rc = skw_walk_records_build(ctx, &ms);
      if (rc) return fail_dev(out, ctx, rc, "skw_walk_records_build");
    }
  }
  long n_total = fb("full") ? (long)V : sh.n_total;
  const long n_local = fb("replica") ? n_total : n_total / sh.ndev;
  const uint64_t id_base = fb("replica") ? 0 : (fb("itl") ? (uint64_t)dev : (uint64_t)dev * n_local);
  const uint64_t id_stride = fb("replica") ? 1 : (fb("itl") ? (uint64_t)sh.ndev : 1);
  // start vertices: the reference starts walker g at vertex g (include/sampler.cuh:494-503)
  std::vector<uint32_t> starts((size_t)std::max<long>(n_local, 1));
  uint32_t* d_starts = nullptr;
  cudaSetDevice(dev);
  if (cudaMalloc(&d_starts, sizeof(uint32_t) * starts.size()) != cudaSuccess)
    return fail_dev(out, nullptr, SKW_ERR_NOMEM, "cudaMalloc(starts)");
  if (fb("randstart")) {
    if (id_stride == 1) rc = skw_generate_starts_device(ctx, n_local, id_base, (uint64_t)fi("seed"), d_starts);
    else {
      std::vector<uint32_t> all((size_t)n_total);
      uint32_t* d_all = nullptr;
      cudaMalloc(&d_all, sizeof(uint32_t) * std::max<long>(n_total, 1));
      rc = skw_generate_starts_device(ctx, n_total, 0, (uint64_t)fi("seed"), d_all);
      skw_ctx_synchronize(ctx);
      cudaMemcpy(all.data(), d_all, sizeof(uint32_t) * n_total, cudaMemcpyDeviceToHost);
      cudaFree(d_all);
      for (long i = 0; i < n_local; ++i) starts[i] = all[id_base + i * id_stride];
      cudaMemcpy(d_starts, starts.data(), sizeof(uint32_t) * n_local, cudaMemcpyHostToDevice);
    }
    if (rc) return fail_dev(out, ctx, rc, "starts");
  } else {
    for (long i = 0; i < n_local; ++i) starts[i] = (uint32_t)((id_base + i * id_stride) % (V ? V : 1));
    cudaMemcpy(d_starts, starts.data(), sizeof(uint32_t) * n_local, cudaMemcpyHostToDevice);
  }
  float ms = 0;
  uint64_t edges = 0;
  uint32_t *d_data = nullptr, *d_len = nullptr;
  if (fb("rw")) {
    skw_walk_params p;
    memset(&p, 0, sizeof p);
    p.app = fb("node2vec") ? SKW_APP_NODE2VEC : (fd("tp") > 0 ? SKW_APP_PPR : SKW_APP_DEEPWALK);
    p.mode = online ? SKW_MODE_ONLINE : SKW_MODE_OFFLINE;
    p.hop_num = (uint32_t)sh.depth + 1;
    p.tp = (float)fd("tp");
    p.p = (float)fd("p");
    p.q = (float)fd("q");
    p.seed = (uint64_t)fi("seed");
    p.walker_base = id_base;
    p.walker_stride = id_stride;
    p.flags = (fb("cache") ? SKW_WALK_CACHE_TABLES : 0) | (bias ? 0 : SKW_WALK_UNBIASED);
    cudaMalloc(&d_data, sizeof(uint32_t) * std::max<long>(n_local, 1) * p.hop_num);
    cudaMalloc(&d_len, sizeof(uint32_t) * std::max<long>(n_local, 1));
    rc = skw_walk_device(ctx, &p, d_starts, n_local, d_data, d_len, &ms, &edges);
    if (rc) return fail_dev(out, ctx, rc, "skw_walk_device");
    if (fb("printresult") && dev == 0) {
      // first three paths, as Jobs_result<RW>::PrintResult does (include/sampler_result.cuh:592-606)
      const long show = std::min<long>(3, n_local);
      std::vector<uint32_t> rows((size_t)show * p.hop_num), lens(show);
      cudaMemcpy(rows.data(), d_data, sizeof(uint32_t) * rows.size(), cudaMemcpyDeviceToHost);
      cudaMemcpy(lens.data(), d_len, sizeof(uint32_t) * show, cudaMemcpyDeviceToHost);
      for (long j = 0; j < show; ++j) {
        printf("\n%ldrd path len %u \n", j, lens[j]);
        for (uint32_t i = 0; i < std::min(lens[j] + 1, p.hop_num); ++i) printf("%u \t", rows[j * p.hop_num + i]);
        printf("\n");
      }
    }
  } else {
    skw_khop_params p;
    memset(&p, 0, sizeof p);
    p.mode = online ? SKW_MODE_ONLINE : SKW_MODE_OFFLINE;
    p.nhops = (uint32_t)sh.depth;
    if (p.nhops > 4) return fail_dev(out, nullptr, SKW_ERR_ARG, "k-hop sampling supports --d up to 4");
    for (uint32_t h = 0; h < p.nhops; ++h) p.fanout[h] = sh.hops[h + 1];
    // the reference copies all neighbours when fan-out >= degree; its online sampler also keeps only
    // draws of columns not drawn before (src/online_sample_new.cu:73-111) unless --replacement asks for
    // independent draws; --bias=0 draws uniformly
    p.flags = SKW_KHOP_TAKE_ALL | (bias ? 0 : SKW_KHOP_UNBIASED);
    if (online && bias && !fb("replacement")) p.flags |= SKW_KHOP_DISTINCT;
    p.seed = (uint64_t)fi("seed");
    uint32_t cells, lens;
    if (skw_khop_layout(&p, &cells, &lens)) return fail_dev(out, nullptr, SKW_ERR_ARG, "bad --k/--d for k-hop sampling");
    cudaMalloc(&d_data, sizeof(uint32_t) * std::max<long>(n_local, 1) * cells);
    cudaMalloc(&d_len, sizeof(uint32_t) * std::max<long>(n_local, 1) * lens);
    const long batches = std::max<long>(1, fi("batches"));
    for (long b = 0; b < batches; ++b) {
      float bms;
      uint64_t bedges;
      p.instance_base = id_base + (uint64_t)b * n_total;
      p.instance_stride = id_stride;
      rc = skw_sample_khop_device(ctx, &p, d_starts, n_local, d_data, d_len, &bms, &bedges);
      if (rc) return fail_dev(out, ctx, rc, "skw_sample_khop_device");
      ms += bms;
      edges += bedges;
    }
    if (fb("printresult") && dev == 0 && p.nhops == 2) {
      // include/sampler_result.cuh:399-420
      const long show = std::min<long>(4, n_local);
      std::vector<uint32_t> rows((size_t)show * cells), sl((size_t)show * lens);
      cudaMemcpy(rows.data(), d_data, sizeof(uint32_t) * rows.size(), cudaMemcpyDeviceToHost);
      cudaMemcpy(sl.data(), d_len, sizeof(uint32_t) * sl.size(), cudaMemcpyDeviceToHost);
      for (long j = 0; j < show; ++j) {
        printf("\n%ldth sample src: %u, 1-hop len: %u \n", j, rows[j * cells], sl[j * lens]);
        printf("\t 1-hop : ");
        for (uint32_t k = 0; k < std::min<uint32_t>(sl[j * lens], 30); ++k) printf("%u \t", rows[j * cells + 1 + k]);
        printf("\n");
      }
    }
  }
  out.time_s = ms * 1e-3f;
  out.sampled = edges;
  LOGV("Device %d sampling time:\t%.6f ratio:\t %.2f MSEPS\n", dev, out.time_s,
       out.time_s > 0 ? edges / out.time_s / 1e6 : 0.0);
#ifdef SKW_HAVE_NCCL
  // results stay on the GPU that produced them (as in the reference); with --gather the per-walker
  // lengths are collected on GPU 0 over NCCL
  if (sh.ndev > 1 && fb("gather") && fb("rw") && !sh.comms.empty() && sh.rv.agree(true)) {
    const size_t cnt = (size_t)std::max<long>(n_local, 1);
    uint32_t* d_all = nullptr;
    if (dev == 0) cudaMalloc(&d_all, sizeof(uint32_t) * cnt * sh.ndev);
    cudaStream_t st;
    cudaStreamCreate(&st);
    // the path rows too (n_local x hop_num per device), when they fit beside GPU 0's own data
    const size_t row_cnt = cnt * (size_t)(fi("d") + 1);
    size_t free_b = 0, total_b = 0;
    if (dev == 0) cudaMemGetInfo(&free_b, &total_b);
    uint32_t* d_rows_all = nullptr;
    int rows_too = dev == 0 && free_b > sizeof(uint32_t) * row_cnt * sh.ndev + (1ull << 30) ? 1 : 0;
    if (dev == 0) sh.gather_rows = rows_too;
    sh.rv.agree(true);  // every device thread sees GPU 0's decision after this point
    rows_too = sh.gather_rows;
    if (rows_too && dev == 0 && cudaMalloc(&d_rows_all, sizeof(uint32_t) * row_cnt * sh.ndev) != cudaSuccess) d_rows_all = nullptr;
    ncclGroupStart();
    ncclSend(d_len, cnt, ncclUint32, 0, sh.comms[dev], st);
    if (dev == 0)
      for (int r = 0; r < sh.ndev; ++r) ncclRecv(d_all + (size_t)r * cnt, cnt, ncclUint32, r, sh.comms[dev], st);
    ncclGroupEnd();
    if (rows_too) {
      ncclGroupStart();
      ncclSend(d_data, row_cnt, ncclUint32, 0, sh.comms[dev], st);
      if (dev == 0 && d_rows_all)
        for (int r = 0; r < sh.ndev; ++r) ncclRecv(d_rows_all + (size_t)r * row_cnt, row_cnt, ncclUint32, r, sh.comms[dev], st);
      ncclGroupEnd();
    }
    cudaStreamSynchronize(st);
    if (dev == 0) {
      sh.gathered_lengths.resize(cnt * sh.ndev);
      cudaMemcpy(sh.gathered_lengths.data(), d_all, sizeof(uint32_t) * cnt * sh.ndev, cudaMemcpyDeviceToHost);
      cudaFree(d_all);
      if (d_rows_all) {
        sh.gathered_paths.resize(row_cnt * sh.ndev);
        cudaMemcpy(sh.gathered_paths.data(), d_rows_all, sizeof(uint32_t) * row_cnt * sh.ndev, cudaMemcpyDeviceToHost);
        cudaFree(d_rows_all);
      }
    }
    cudaStreamDestroy(st);
  }
#endif
  cudaFree(d_starts);
  cudaFree(d_data);
  cudaFree(d_len);
  return 0;
}

}  // namespace

int main(int argc, char** argv) {
  define_flags();
  if (parse_flags(argc, argv)) return 1;
  // presets, src/main.cu:156-184
  const bool d_given = was_set("d");
  if (fb("node2vec") || fb("deepwalk") || fb("ppr")) {
    setb("rw", true);
    seti("k", 1);
    if (!d_given) seti("d", 100);
    if (fb("ppr") && !was_set("tp")) g_flags.at("tp").value = "0.15";
  }
  if (fb("sage")) {
    setb("rw", false);
    seti("d", 2);
  }
  if (fs("input").empty() && fi("rmat_scale") <= 0) {
    fprintf(stderr, "need --input <file.gr> (or --rmat_scale N for a synthetic graph)\n");
    return 1;
  }
  Shared sh;
  sh.ndev = (int)std::max<long>(1, fi("ngpu"));
  sh.n_total = fi("n");
  sh.depth = (int)fi("d");
  sh.hops.assign(sh.depth + 1, (uint32_t)fi("k"));
  sh.hops[0] = 1;
  if (fb("sage")) {
    sh.hops[1] = 25;
    sh.hops[2] = 10;
  }
  int have = 0;
  if (cudaGetDeviceCount(&have) != cudaSuccess || have < sh.ndev) {
    fprintf(stderr, "--ngpu %d but %d CUDA device(s) are visible\n", sh.ndev, have);
    return 1;
  }
  // graph name first, as Graph::ReadGraphGR prints it (include/graph.cuh:181-192)
  {
    const std::string& path = fs("input");
    std::string token = path.empty() ? "rmat" + fs("rmat_scale") : path.substr(path.rfind('/') + 1);
    if (fb("csv")) printf("%s,", token.c_str());
    else if (!fb("v")) printf("%s\n", token.c_str());
  }
#ifdef SKW_HAVE_NCCL
  if (sh.ndev > 1) {
    sh.comms.resize(sh.ndev);
    std::vector<int> devs(sh.ndev);
    for (int i = 0; i < sh.ndev; ++i) devs[i] = i;
    if (ncclCommInitAll(sh.comms.data(), sh.ndev, devs.data()) != ncclSuccess) {
      fprintf(stderr, "ncclCommInitAll failed; continuing with replicated builds and no result gather\n");
      sh.comms.clear();
    }
  }
#endif
  std::vector<DevResult> res(sh.ndev);
  std::vector<std::thread> th;
  sh.rv.ndev = sh.ndev;
  for (int dev = 0; dev < sh.ndev; ++dev)
    th.emplace_back([&, dev] {
      run_device(dev, sh, res[dev]);
      sh.rv.leave();
    });
  for (auto& t : th) t.join();
#ifdef SKW_HAVE_NCCL
  for (auto c : sh.comms) ncclCommDestroy(c);
#endif
  for (int dev = 0; dev < sh.ndev; ++dev)
    if (res[dev].rc) {
      fprintf(stderr, "device %d: %s\n", dev, res[dev].err.c_str());
      return 2;
    }
  // MSEPS = sum of sampled edges / max time / 1e6, src/main.cu:377-394
  float table_ms = 0, max_s = 0;
  uint64_t sampled = 0;
  for (auto& r : res) {
    table_ms = std::max(table_ms, r.table_ms);
    max_s = std::max(max_s, r.time_s);
    sampled += r.sampled;
  }
  const double mseps = max_s > 0 ? sampled / (double)max_s / 1e6 : 0.0;
  LOGV("sampled_edges %llu\n", (unsigned long long)sampled);  // as src/offline_walk.cu:226 logs it
  if (!sh.gathered_lengths.empty()) {
    uint64_t total = 0;
    for (uint32_t l : sh.gathered_lengths) total += l;
    LOGV("gathered %zu walk lengths on GPU 0 over NCCL, sum %llu\n", sh.gathered_lengths.size(),
         (unsigned long long)total);
    if (!sh.gathered_paths.empty()) {
      // every gathered row starts with a vertex and holds length + 1 cells: count them as a check
      const size_t hop = (size_t)fi("d") + 1;
      uint64_t cells = 0;
      for (size_t w = 0; w < sh.gathered_lengths.size(); ++w) cells += std::min<size_t>(sh.gathered_lengths[w] + 1, hop);
      LOGV("gathered %zu path rows x %zu cells on GPU 0 over NCCL, %llu cells hold a vertex\n",
           sh.gathered_paths.size() / hop, hop, (unsigned long long)cells);
    }
  }
  const bool offline_biased = !fb("ol") && fb("bias");
  if (fb("csv")) {
    if (offline_biased) printf("%0.2f,\t", table_ms);
    printf("%0.2f,\t", max_s * 1000);
    printf("%0.2f,\n", mseps);
  } else {
    if (offline_biased)
      for (int i = 0; i < sh.ndev; ++i) printf("%0.2f\t", i == sh.ndev - 1 ? table_ms : 0.0f);
    printf("\n");
    for (int i = 0; i < sh.ndev; ++i) printf("%0.2f\t", i == sh.ndev - 1 ? max_s * 1000 : 0.0f);
    printf("\n");
    for (int i = 0; i < sh.ndev; ++i) printf("%0.2f\t", i == sh.ndev - 1 ? mseps : 0.0);
    printf("\n");
  }
  return 0;
}
