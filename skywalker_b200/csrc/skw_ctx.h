// Host-side state behind the opaque skw_ctx handle, and the helpers every translation unit of
// the library uses to report errors and count launches.
#pragma once
#include <cuda_runtime.h>
#include <stdint.h>

#include <string>

#include "../../include/skywalker_b200.h"
#include "skw_device.cuh"

namespace skw {

// Spare slots allocated past the table's E entries (room for the padded last chunk of an in-place
// all-gather over up to 1024 ranks).
constexpr uint32_t kSlotSlack = 1024;

// Largest degree the shared-memory CTA builder takes (12 bytes of list state per edge).
constexpr uint32_t kCtaSmemMaxDegree = 4096;

}  // namespace skw

struct skw_ctx {
  int device = 0;
  int sm_count = 0;
  cudaStream_t own_stream = nullptr;
  cudaStream_t stream = nullptr;
  cudaStream_t side_stream = nullptr;  // result copies that overlap kernels of `stream`
  cudaStream_t copy_stream = nullptr;  // skw_walk_packed: the packed rows of each slice
  // skw_walk_packed, per slice: rows packed; cell count on the host; start and end of the walk
  static constexpr int kPackSlices = 8;
  cudaEvent_t pk_ready[kPackSlices] = {}, pk_tot[kPackSlices] = {}, pk_t0[kPackSlices] = {}, pk_t1[kPackSlices] = {},
              pk_in[kPackSlices] = {};
  uint64_t* d_tot = nullptr;  // cells each slice's packed result needs
  uint64_t* h_tot = nullptr;  // pinned mirror
  cudaEvent_t ev0 = nullptr, ev1 = nullptr;
  // the degree-class builders of one build run side by side: classes 257+ on streams of their own,
  // forked from and joined back into `stream` by events
  static constexpr int kBuilderStreams = 4;
  cudaStream_t bstream[kBuilderStreams] = {nullptr, nullptr, nullptr, nullptr};
  cudaEvent_t bfork = nullptr, bjoin[kBuilderStreams] = {nullptr, nullptr, nullptr, nullptr};
  std::string err;
  uint64_t launches = 0;

  // resident CSR
  uint32_t V = 0;
  uint64_t E = 0;
  uint32_t max_degree = 0;
  uint32_t* xadj = nullptr;
  uint32_t* adjncy = nullptr;
  float* adjwgt = nullptr;
  bool owns_graph = false;
  bool owns_weights = false;

  // alias table
  skw::Slot* slots = nullptr;
  uint8_t* valid = nullptr;
  bool table_ready = false;
  // optional fused walk records (32 B per edge slot) and per-vertex {offset, usable degree}
  void* records = nullptr;
  void* vinfo = nullptr;
  void* vbits = nullptr;  // one bit per vertex: usable degree != 0
  bool records_ready = false;  // set once records, vinfo and vbits were all written
  bool records_all_usable = false;  // ... and no vertex with out-edges lacks a usable table

  // device error word (4 x u32) and its pinned host mirror
  uint32_t* d_err = nullptr;
  uint32_t* h_err = nullptr;
  // pinned scalar for 64-bit reductions read back after a launch
  uint64_t* d_sum = nullptr;
  uint64_t* h_sum = nullptr;

  // builder scratch, grown on demand
  uint32_t* worklist = nullptr;      // V entries, vertices grouped by degree class
  size_t worklist_cap = 0;
  uint32_t* cls_counts = nullptr;    // per degree class: count, fill cursor, base in the work list
  void* cta_scratch = nullptr;       // slabs of the global-memory CTA builder
  size_t cta_scratch_bytes = 0;

  // online mode: per-frontier work lists (one per degree class) and the claim stamps that make
  // every distinct frontier vertex be built once per round
  uint32_t* frontier_lists = nullptr;
  size_t frontier_lists_bytes = 0;
  uint32_t* frontier_cls = nullptr;  // same layout as cls_counts
  uint32_t* stamp = nullptr;         // V entries, last round that claimed the vertex
  uint32_t stamp_round = 0;
  // online direct walks: per-vertex memo of {call stamp, largest weight, total quantised weight}
  void* prep_memo = nullptr;
  uint32_t prep_stamp = 0;
  void* prep_ckpt = nullptr;  // prefix-sum checkpoints of long lists, valid together with the memo entry

  // skw_walk with host rows, large batches: pinned staging for the packed result and the host threads
  // that scatter it into the caller's matrix
  uint32_t* h_pack = nullptr;
  size_t h_pack_cells = 0;
  void* host_pool = nullptr;  // skw::HostPool

  // staging buffers of the host-pointer entry points, grown on demand
  static constexpr int kStages = 13;
  void* stage[kStages] = {};
  size_t stage_bytes[kStages] = {};
};

namespace skw {

int fail(skw_ctx* ctx, int code, const char* fmt, ...);
// after the CSR pointers are set: compute max_degree
int finish_graph(skw_ctx* ctx);
// allocate slots[E] / valid[V] if absent
int alloc_table(skw_ctx* ctx);
// forget the fused walk records (they are derived from the table and die with it)
void drop_records(skw_ctx* ctx);
int fail_cuda(skw_ctx* ctx, cudaError_t e, const char* what, const char* file, int line);
void set_global_error(const char* msg);

// Grow-only device buffer.
int ensure_bytes(skw_ctx* ctx, void** p, size_t* cap, size_t want);
// Zero the device error word before a group of launches / check it after synchronising.
int err_reset(skw_ctx* ctx);
int err_check(skw_ctx* ctx, const char* where);

struct DeviceGuard {
  int prev = -1;
  explicit DeviceGuard(int dev) {
    cudaGetDevice(&prev);
    if (prev != dev) cudaSetDevice(dev);
    else prev = -1;
  }
  ~DeviceGuard() {
    if (prev >= 0) cudaSetDevice(prev);
  }
};

}  // namespace skw

#define SKW_CUDA(ctx, call)                                                          \
  do {                                                                               \
    cudaError_t e__ = (call);                                                        \
    if (e__ != cudaSuccess) return skw::fail_cuda((ctx), e__, #call, __FILE__, __LINE__); \
  } while (0)

// Count a kernel launch and surface a launch-configuration error at once.
#define SKW_LAUNCHED(ctx)                                                            \
  do {                                                                               \
    (ctx)->launches++;                                                               \
    cudaError_t e__ = cudaGetLastError();                                            \
    if (e__ != cudaSuccess) return skw::fail_cuda((ctx), e__, "kernel launch", __FILE__, __LINE__); \
  } while (0)
