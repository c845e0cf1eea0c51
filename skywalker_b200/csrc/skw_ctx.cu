// Context, resident graph, table import/export and the Galois .gr reader.
#include <algorithm>
#include <cstdarg>
#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <mutex>
#include <vector>

#include "skw_ctx.h"
#include "skw_hostpool.h"

namespace skw {

static std::mutex g_err_mu;
static std::string g_err;

void set_global_error(const char* msg) {
  std::lock_guard<std::mutex> lk(g_err_mu);
  g_err = msg;
}

int fail(skw_ctx* ctx, int code, const char* fmt, ...) {
  char buf[512];
  va_list ap;
  va_start(ap, fmt);
  vsnprintf(buf, sizeof buf, fmt, ap);
  va_end(ap);
  if (ctx) ctx->err = buf;
  else set_global_error(buf);
  return code;
}

int fail_cuda(skw_ctx* ctx, cudaError_t e, const char* what, const char* file, int line) {
  const char* base = strrchr(file, '/');
  return fail(ctx, SKW_ERR_CUDA, "%s: %s (%s:%d)", what, cudaGetErrorString(e),
              base ? base + 1 : file, line);
}

int ensure_bytes(skw_ctx* ctx, void** p, size_t* cap, size_t want) {
  if (*cap >= want && *p) return SKW_OK;
  if (*p) SKW_CUDA(ctx, cudaFree(*p));
  *p = nullptr;
  *cap = 0;
  if (want == 0) want = 256;
  SKW_CUDA(ctx, cudaMalloc(p, want));
  *cap = want;
  return SKW_OK;
}

int err_reset(skw_ctx* ctx) {
  SKW_CUDA(ctx, cudaMemsetAsync(ctx->d_err, 0, 4 * sizeof(uint32_t), ctx->stream));
  return SKW_OK;
}

int err_check(skw_ctx* ctx, const char* where) {
  SKW_CUDA(ctx, cudaMemcpyAsync(ctx->h_err, ctx->d_err, 4 * sizeof(uint32_t),
                                cudaMemcpyDeviceToHost, ctx->stream));
  SKW_CUDA(ctx, cudaStreamSynchronize(ctx->stream));
  if (ctx->h_err[0] != DEV_OK) {
    static const char* names[] = {"ok", "index out of range", "bounded wait ran out",
                                  "capacity exceeded", "construction invariant broken"};
    const uint32_t c = ctx->h_err[0];
    return fail(ctx, SKW_ERR_DEVICE, "%s: device error %u (%s), detail %u %u %u", where, c,
                c < 5 ? names[c] : "?", ctx->h_err[1], ctx->h_err[2], ctx->h_err[3]);
  }
  return SKW_OK;
}

static void free_graph(skw_ctx* ctx) {
  if (ctx->owns_graph) {
    cudaFree(ctx->xadj);
    cudaFree(ctx->adjncy);
  }
  if (ctx->owns_weights) cudaFree(ctx->adjwgt);
  ctx->xadj = ctx->adjncy = nullptr;
  ctx->adjwgt = nullptr;
  ctx->owns_graph = ctx->owns_weights = false;
  cudaFree(ctx->slots);
  cudaFree(ctx->valid);
  cudaFree(ctx->stamp);
  cudaFree(ctx->prep_memo);
  cudaFree(ctx->prep_ckpt);
  ctx->prep_ckpt = nullptr;
  ctx->prep_memo = nullptr;
  ctx->prep_stamp = 0;
  cudaFree(ctx->records);
  cudaFree(ctx->vinfo);
  cudaFree(ctx->vbits);
  ctx->records = nullptr;
  ctx->vinfo = nullptr;
  ctx->vbits = nullptr;
  ctx->records_ready = false;
  ctx->stamp = nullptr;
  ctx->stamp_round = 0;
  ctx->slots = nullptr;
  ctx->valid = nullptr;
  ctx->table_ready = false;
  ctx->V = 0;
  ctx->E = 0;
  ctx->max_degree = 0;
}

__global__ void max_degree_kernel(const uint32_t* __restrict__ xadj, uint32_t V,
                                  uint32_t* __restrict__ out) {
  uint32_t m = 0;
  for (size_t v = blockIdx.x * (size_t)blockDim.x + threadIdx.x; v < V;
       v += (size_t)gridDim.x * blockDim.x)
    m = max(m, xadj[v + 1] - xadj[v]);
  for (int o = 16; o; o >>= 1) m = max(m, __shfl_xor_sync(0xFFFFFFFFu, m, o));
  if ((threadIdx.x & 31) == 0 && m) atomicMax(out, m);
}

__global__ void fill_ones_kernel(float* __restrict__ w, size_t n) {
  for (size_t i = blockIdx.x * (size_t)blockDim.x + threadIdx.x; i < n;
       i += (size_t)gridDim.x * blockDim.x)
    w[i] = 1.0f;
}

// Weight of every edge = out-degree of its source (reference --dw, include/graph.cuh:299-310).
__global__ void fill_degree_weights_kernel(const uint32_t* __restrict__ xadj, uint32_t V,
                                           float* __restrict__ w) {
  const uint32_t lane = threadIdx.x & 31;
  const size_t warp = (blockIdx.x * (size_t)blockDim.x + threadIdx.x) >> 5;
  const size_t nwarps = ((size_t)gridDim.x * blockDim.x) >> 5;
  for (size_t v = warp; v < V; v += nwarps) {
    const uint32_t b = xadj[v], e = xadj[v + 1];
    const float d = (float)(e - b);
    for (uint32_t i = b + lane; i < e; i += 32) w[i] = d;
  }
}

// Seeded uniform weight in [0, range): the reproducible stand-in for the reference's
// rand() / (RAND_MAX / weightrange) with srand(0) (include/graph.cuh:210-219).
__global__ void fill_random_weights_kernel(float* __restrict__ w, size_t n, uint64_t seed,
                                           float range) {
  for (size_t i = blockIdx.x * (size_t)blockDim.x + threadIdx.x; i < n;
       i += (size_t)gridDim.x * blockDim.x) {
    const Rand4 r = philox_tagged(seed, TAG_WGHT, i, 1, 0);
    w[i] = u01(r.x) * range;
  }
}

// Structural check of a CSR handed in by a caller: offsets non-decreasing and at most E, every
// destination below V.  Every kernel of the library indexes with these values unchecked, so a bad
// array is refused here (error word, no fault) instead of being walked.
__global__ void __launch_bounds__(256) validate_csr_kernel(const uint32_t* __restrict__ xadj,
                                                           const uint32_t* __restrict__ adjncy, uint32_t V,
                                                           uint64_t E, uint32_t* __restrict__ err) {
  const size_t T = (size_t)gridDim.x * blockDim.x, t0 = blockIdx.x * (size_t)blockDim.x + threadIdx.x;
  for (size_t v = t0; v < V; v += T) {
    const uint32_t a = xadj[v], b = xadj[v + 1];
    if (a > b || b > E) dev_fail(err, DEV_ERR_INDEX, (uint32_t)v, a, b);
  }
  if (t0 == 0 && (xadj[0] != 0 || xadj[V] != (uint32_t)E)) dev_fail(err, DEV_ERR_INDEX, V, xadj[0], xadj[V]);
  for (size_t e = t0; e < E; e += T) {
    const uint32_t d = adjncy[e];
    if (d >= V) dev_fail(err, DEV_ERR_INDEX, d, (uint32_t)e, 21);
  }
}

int validate_graph(skw_ctx* ctx, const char* who) {
  int rc = err_reset(ctx);
  if (rc != SKW_OK) return rc;
  validate_csr_kernel<<<ctx->sm_count * 8, 256, 0, ctx->stream>>>(ctx->xadj, ctx->adjncy, ctx->V, ctx->E, ctx->d_err);
  SKW_LAUNCHED(ctx);
  rc = err_check(ctx, who);
  if (rc == SKW_ERR_DEVICE) {
    const std::string why = ctx->err;
    free_graph(ctx);
    return fail(ctx, SKW_ERR_ARG, "%s: the CSR is malformed (offsets must be non-decreasing from 0 to E, destinations below V) -- %s",
                who, why.c_str());
  }
  return rc;
}

// Every slot starts as {prob = -1, alias = 0}: "no usable table here".  A walker or k-hop draw that
// meets such a slot ends, so vertices outside the range a sliced build has covered so far (or whose
// slice has not arrived yet) are dead ends rather than reads of uninitialised memory.
__global__ void __launch_bounds__(256) fill_unbuilt_slots_kernel(Slot* __restrict__ slots, size_t n) {
  for (size_t i = blockIdx.x * (size_t)blockDim.x + threadIdx.x; i < n; i += (size_t)gridDim.x * blockDim.x)
    slots[i] = Slot{-1.0f, 0u};
}

// Check of a table that did not come from the builders (import, checkpoint): every alias must point
// inside its vertex's list and every prob must be -1 (invalid vertex) or in [0, 1].
__global__ void __launch_bounds__(256) validate_table_kernel(const uint32_t* __restrict__ xadj,
                                                             const Slot* __restrict__ slots, uint32_t V,
                                                             uint32_t* __restrict__ err) {
  const uint32_t lane = threadIdx.x & 31;
  const size_t warp = (blockIdx.x * (size_t)blockDim.x + threadIdx.x) >> 5;
  const size_t nwarps = ((size_t)gridDim.x * blockDim.x) >> 5;
  for (size_t v = warp; v < V; v += nwarps) {
    const uint32_t off = xadj[v], deg = xadj[v + 1] - off;
    for (uint32_t i = lane; i < deg; i += 32) {
      const Slot s = slots[(size_t)off + i];
      const bool prob_ok = s.prob == -1.0f || (s.prob >= 0.0f && s.prob <= 1.0f);
      if (s.alias >= deg || !prob_ok) dev_fail(err, DEV_ERR_INDEX, (uint32_t)v, i, s.alias);
    }
  }
}

int validate_table(skw_ctx* ctx, const char* who) {
  int rc = err_reset(ctx);
  if (rc != SKW_OK) return rc;
  if (ctx->V) {
    validate_table_kernel<<<ctx->sm_count * 8, 256, 0, ctx->stream>>>(ctx->xadj, ctx->slots, ctx->V, ctx->d_err);
    SKW_LAUNCHED(ctx);
  }
  rc = err_check(ctx, who);
  if (rc == SKW_ERR_DEVICE) {
    const std::string why = ctx->err;
    return fail(ctx, SKW_ERR_ARG, "%s: the table does not fit the resident graph (an alias outside its vertex's list or a prob "
                "outside [0,1]) -- %s", who, why.c_str());
  }
  return rc;
}

// 64-bit fingerprint of the offset array: sum over v of mix(v, xadj[v]).  Stored in a table
// checkpoint so that a table written for another graph with the same V and E is refused.
__global__ void __launch_bounds__(256) xadj_fingerprint_kernel(const uint32_t* __restrict__ xadj, uint32_t V,
                                                               unsigned long long* __restrict__ out) {
  unsigned long long acc = 0;
  for (size_t v = blockIdx.x * (size_t)blockDim.x + threadIdx.x; v <= V; v += (size_t)gridDim.x * blockDim.x) {
    unsigned long long x = ((unsigned long long)v << 32) ^ xadj[v];
    x ^= x >> 33;
    x *= 0xff51afd7ed558ccdull;
    x ^= x >> 33;
    x *= 0xc4ceb9fe1a85ec53ull;
    x ^= x >> 33;
    acc += x;
  }
  for (int o = 16; o; o >>= 1) acc += __shfl_xor_sync(0xFFFFFFFFu, acc, o);
  if ((threadIdx.x & 31) == 0) atomicAdd(out, acc);
}

static int xadj_fingerprint(skw_ctx* ctx, uint64_t* out) {
  SKW_CUDA(ctx, cudaMemsetAsync(ctx->d_sum, 0, sizeof(uint64_t), ctx->stream));
  xadj_fingerprint_kernel<<<ctx->sm_count * 4, 256, 0, ctx->stream>>>(ctx->xadj, ctx->V,
                                                                      reinterpret_cast<unsigned long long*>(ctx->d_sum));
  SKW_LAUNCHED(ctx);
  SKW_CUDA(ctx, cudaMemcpyAsync(ctx->h_sum, ctx->d_sum, sizeof(uint64_t), cudaMemcpyDeviceToHost, ctx->stream));
  SKW_CUDA(ctx, cudaStreamSynchronize(ctx->stream));
  *out = *ctx->h_sum;
  return SKW_OK;
}

int finish_graph(skw_ctx* ctx) {
  SKW_CUDA(ctx, cudaMemsetAsync(ctx->d_sum, 0, sizeof(uint64_t), ctx->stream));
  if (ctx->V) {
    max_degree_kernel<<<ctx->sm_count * 4, 256, 0, ctx->stream>>>(
        ctx->xadj, ctx->V, reinterpret_cast<uint32_t*>(ctx->d_sum));
    SKW_LAUNCHED(ctx);
  }
  SKW_CUDA(ctx, cudaMemcpyAsync(ctx->h_sum, ctx->d_sum, sizeof(uint64_t), cudaMemcpyDeviceToHost,
                                ctx->stream));
  SKW_CUDA(ctx, cudaStreamSynchronize(ctx->stream));
  ctx->max_degree = (uint32_t)*ctx->h_sum;
  return SKW_OK;
}

void drop_records(skw_ctx* ctx) {
  ctx->records_ready = false;
  if (ctx->records || ctx->vinfo) cudaStreamSynchronize(ctx->stream);
  cudaFree(ctx->records);
  cudaFree(ctx->vinfo);
  cudaFree(ctx->vbits);
  ctx->records = nullptr;
  ctx->vinfo = nullptr;
  ctx->vbits = nullptr;
}

int alloc_table(skw_ctx* ctx) {
  // kSlotSlack spare entries let a multi-GPU caller all-gather the table in equal chunks in place
  if (!ctx->slots) {
    SKW_CUDA(ctx, cudaMalloc(&ctx->slots, sizeof(Slot) * (ctx->E + kSlotSlack)));
    fill_unbuilt_slots_kernel<<<ctx->sm_count * 8, 256, 0, ctx->stream>>>(ctx->slots, (size_t)ctx->E + kSlotSlack);
    SKW_LAUNCHED(ctx);
  }
  if (!ctx->valid) {
    SKW_CUDA(ctx, cudaMalloc(&ctx->valid, ctx->V ? ctx->V : 1));
    SKW_CUDA(ctx, cudaMemsetAsync(ctx->valid, 0, ctx->V ? ctx->V : 1, ctx->stream));
  }
  return SKW_OK;
}

}  // namespace skw

using namespace skw;

extern "C" {

const char* skw_version(void) { return "0.1"; }

const char* skw_last_global_error(void) {
  std::lock_guard<std::mutex> lk(g_err_mu);
  static thread_local std::string copy;
  copy = g_err;
  return copy.c_str();
}

const char* skw_last_error(const skw_ctx* ctx) { return ctx ? ctx->err.c_str() : ""; }

int skw_ctx_create(int device, skw_ctx** out) {
  if (!out) return fail(nullptr, SKW_ERR_ARG, "skw_ctx_create: out is null");
  *out = nullptr;
  int count = 0;
  cudaError_t e = cudaGetDeviceCount(&count);
  if (e != cudaSuccess || count == 0)
    return fail(nullptr, SKW_ERR_CUDA, "skw_ctx_create: no CUDA device (%s); this library has no CPU path",
                e == cudaSuccess ? "device count is 0" : cudaGetErrorString(e));
  if (device < 0 || device >= count)
    return fail(nullptr, SKW_ERR_ARG, "skw_ctx_create: device %d out of range [0,%d)", device, count);
  skw_ctx* ctx = new skw_ctx();
  ctx->device = device;
#define CK(call)                                                                 \
  do {                                                                           \
    cudaError_t e2 = (call);                                                     \
    if (e2 != cudaSuccess) {                                                     \
      fail(nullptr, SKW_ERR_CUDA, "skw_ctx_create: %s: %s", #call, cudaGetErrorString(e2)); \
      skw_ctx_destroy(ctx);                                                      \
      return SKW_ERR_CUDA;                                                       \
    }                                                                            \
  } while (0)
  CK(cudaSetDevice(device));
  cudaDeviceProp prop;
  CK(cudaGetDeviceProperties(&prop, device));
  ctx->sm_count = prop.multiProcessorCount;
  CK(cudaStreamCreateWithFlags(&ctx->own_stream, cudaStreamNonBlocking));
  CK(cudaStreamCreateWithFlags(&ctx->side_stream, cudaStreamNonBlocking));
  CK(cudaStreamCreateWithFlags(&ctx->copy_stream, cudaStreamNonBlocking));
  ctx->stream = ctx->own_stream;
  for (int i = 0; i < skw_ctx::kBuilderStreams; ++i) {
    CK(cudaStreamCreateWithFlags(&ctx->bstream[i], cudaStreamNonBlocking));
    CK(cudaEventCreateWithFlags(&ctx->bjoin[i], cudaEventDisableTiming));
  }
  CK(cudaEventCreateWithFlags(&ctx->bfork, cudaEventDisableTiming));
  CK(cudaEventCreate(&ctx->ev0));
  CK(cudaEventCreate(&ctx->ev1));
  // two error records of four words: [0..4) reset and checked by every call, [4..8) owned by the
  // packing pipeline of skw_walk_packed, which spans several such calls
  CK(cudaMalloc(&ctx->d_err, 8 * sizeof(uint32_t)));
  CK(cudaMemset(ctx->d_err, 0, 8 * sizeof(uint32_t)));
  CK(cudaMallocHost(&ctx->h_err, 8 * sizeof(uint32_t)));
  for (int i = 0; i < skw_ctx::kPackSlices; ++i) {
    CK(cudaEventCreateWithFlags(&ctx->pk_ready[i], cudaEventDisableTiming));
    CK(cudaEventCreateWithFlags(&ctx->pk_in[i], cudaEventDisableTiming));
    CK(cudaEventCreateWithFlags(&ctx->pk_tot[i], cudaEventDisableTiming));
    CK(cudaEventCreate(&ctx->pk_t0[i]));
    CK(cudaEventCreate(&ctx->pk_t1[i]));
  }
  CK(cudaMalloc(&ctx->d_tot, skw_ctx::kPackSlices * sizeof(uint64_t)));
  CK(cudaMallocHost(&ctx->h_tot, skw_ctx::kPackSlices * sizeof(uint64_t)));
  CK(cudaMalloc(&ctx->d_sum, 4 * sizeof(uint64_t)));
  CK(cudaMemset(ctx->d_sum, 0, 4 * sizeof(uint64_t)));
  CK(cudaMallocHost(&ctx->h_sum, 4 * sizeof(uint64_t)));
  CK(cudaMalloc(&ctx->cls_counts, 64 * sizeof(uint32_t)));
  CK(cudaMalloc(&ctx->frontier_cls, 64 * sizeof(uint32_t)));
#undef CK
  *out = ctx;
  return SKW_OK;
}

void skw_ctx_destroy(skw_ctx* ctx) {
  if (!ctx) return;
  cudaSetDevice(ctx->device);
  if (ctx->own_stream) cudaStreamSynchronize(ctx->own_stream);
  free_graph(ctx);
  cudaFree(ctx->d_err);
  cudaFreeHost(ctx->h_err);
  cudaFree(ctx->d_sum);
  cudaFreeHost(ctx->h_sum);
  cudaFree(ctx->worklist);
  cudaFree(ctx->cls_counts);
  cudaFree(ctx->cta_scratch);
  cudaFree(ctx->frontier_lists);
  cudaFree(ctx->frontier_cls);
  for (int i = 0; i < skw_ctx::kStages; ++i) cudaFree(ctx->stage[i]);
  if (ctx->h_pack) cudaFreeHost(ctx->h_pack);
  delete static_cast<skw::HostPool*>(ctx->host_pool);
  cudaFree(ctx->d_tot);
  cudaFreeHost(ctx->h_tot);
  if (ctx->ev0) cudaEventDestroy(ctx->ev0);
  if (ctx->ev1) cudaEventDestroy(ctx->ev1);
  if (ctx->own_stream) cudaStreamDestroy(ctx->own_stream);
  if (ctx->side_stream) cudaStreamDestroy(ctx->side_stream);
  if (ctx->copy_stream) cudaStreamDestroy(ctx->copy_stream);
  for (int i = 0; i < skw_ctx::kBuilderStreams; ++i) {
    if (ctx->bstream[i]) cudaStreamDestroy(ctx->bstream[i]);
    if (ctx->bjoin[i]) cudaEventDestroy(ctx->bjoin[i]);
  }
  if (ctx->bfork) cudaEventDestroy(ctx->bfork);
  for (int i = 0; i < skw_ctx::kPackSlices; ++i) {
    if (ctx->pk_ready[i]) cudaEventDestroy(ctx->pk_ready[i]);
    if (ctx->pk_in[i]) cudaEventDestroy(ctx->pk_in[i]);
    if (ctx->pk_tot[i]) cudaEventDestroy(ctx->pk_tot[i]);
    if (ctx->pk_t0[i]) cudaEventDestroy(ctx->pk_t0[i]);
    if (ctx->pk_t1[i]) cudaEventDestroy(ctx->pk_t1[i]);
  }
  delete ctx;
}

int skw_ctx_set_stream(skw_ctx* ctx, void* cuda_stream) {
  if (!ctx) return SKW_ERR_ARG;
  ctx->stream = cuda_stream ? static_cast<cudaStream_t>(cuda_stream) : ctx->own_stream;
  return SKW_OK;
}

int skw_ctx_synchronize(skw_ctx* ctx) {
  if (!ctx) return SKW_ERR_ARG;
  DeviceGuard g(ctx->device);
  SKW_CUDA(ctx, cudaStreamSynchronize(ctx->stream));
  return SKW_OK;
}

uint64_t skw_ctx_kernel_launches(const skw_ctx* ctx) { return ctx ? ctx->launches : 0; }

int skw_graph_upload(skw_ctx* ctx, uint32_t V, uint64_t E, const uint32_t* h_xadj,
                     const uint32_t* h_adjncy, const float* h_adjwgt) {
  if (!ctx) return SKW_ERR_ARG;
  if (!h_xadj || (E && !h_adjncy)) return fail(ctx, SKW_ERR_ARG, "skw_graph_upload: null CSR array");
  if (E > 0xFFFFFFFFull) return fail(ctx, SKW_ERR_ARG, "skw_graph_upload: E must fit 32 bits");
  if (V == 0xFFFFFFFFu) return fail(ctx, SKW_ERR_ARG, "skw_graph_upload: V too large");
  if (h_xadj[0] != 0 || h_xadj[V] != E)
    return fail(ctx, SKW_ERR_ARG, "skw_graph_upload: xadj[0] must be 0 and xadj[V] must equal E");
  DeviceGuard g(ctx->device);
  free_graph(ctx);
  SKW_CUDA(ctx, cudaMalloc(&ctx->xadj, sizeof(uint32_t) * ((size_t)V + 1)));
  SKW_CUDA(ctx, cudaMalloc(&ctx->adjncy, sizeof(uint32_t) * (E ? E : 1)));
  SKW_CUDA(ctx, cudaMalloc(&ctx->adjwgt, sizeof(float) * (E ? E : 1)));
  ctx->owns_graph = ctx->owns_weights = true;
  ctx->V = V;
  ctx->E = E;
  SKW_CUDA(ctx, cudaMemcpyAsync(ctx->xadj, h_xadj, sizeof(uint32_t) * ((size_t)V + 1),
                                cudaMemcpyHostToDevice, ctx->stream));
  if (E) {
    SKW_CUDA(ctx, cudaMemcpyAsync(ctx->adjncy, h_adjncy, sizeof(uint32_t) * E,
                                  cudaMemcpyHostToDevice, ctx->stream));
    if (h_adjwgt) {
      SKW_CUDA(ctx, cudaMemcpyAsync(ctx->adjwgt, h_adjwgt, sizeof(float) * E,
                                    cudaMemcpyHostToDevice, ctx->stream));
    } else {
      fill_ones_kernel<<<ctx->sm_count * 4, 256, 0, ctx->stream>>>(ctx->adjwgt, E);
      SKW_LAUNCHED(ctx);
    }
  }
  int rc = validate_graph(ctx, "skw_graph_upload");
  if (rc != SKW_OK) return rc;
  return finish_graph(ctx);
}

int skw_graph_adopt_device(skw_ctx* ctx, uint32_t V, uint64_t E, const uint32_t* d_xadj,
                           const uint32_t* d_adjncy, const float* d_adjwgt) {
  if (!ctx) return SKW_ERR_ARG;
  if (!d_xadj || (E && !d_adjncy))
    return fail(ctx, SKW_ERR_ARG, "skw_graph_adopt_device: null CSR array");
  if (E > 0xFFFFFFFFull) return fail(ctx, SKW_ERR_ARG, "skw_graph_adopt_device: E must fit 32 bits");
  DeviceGuard g(ctx->device);
  free_graph(ctx);
  ctx->xadj = const_cast<uint32_t*>(d_xadj);
  ctx->adjncy = const_cast<uint32_t*>(d_adjncy);
  ctx->adjwgt = const_cast<float*>(d_adjwgt);
  ctx->V = V;
  ctx->E = E;
  if (!d_adjwgt) {
    SKW_CUDA(ctx, cudaMalloc(&ctx->adjwgt, sizeof(float) * (E ? E : 1)));
    ctx->owns_weights = true;
    fill_ones_kernel<<<ctx->sm_count * 4, 256, 0, ctx->stream>>>(ctx->adjwgt, E);
    SKW_LAUNCHED(ctx);
  }
  int rc = validate_graph(ctx, "skw_graph_adopt_device");
  if (rc != SKW_OK) return rc;
  return finish_graph(ctx);
}

int skw_graph_info(const skw_ctx* ctx, uint32_t* V, uint64_t* E, uint32_t* max_degree) {
  if (!ctx) return SKW_ERR_ARG;
  if (V) *V = ctx->V;
  if (E) *E = ctx->E;
  if (max_degree) *max_degree = ctx->max_degree;
  return SKW_OK;
}

int skw_graph_download(skw_ctx* ctx, uint32_t* h_xadj, uint32_t* h_adjncy, float* h_adjwgt) {
  if (!ctx) return SKW_ERR_ARG;
  if (!ctx->xadj) return fail(ctx, SKW_ERR_STATE, "skw_graph_download: no graph resident");
  DeviceGuard g(ctx->device);
  if (h_xadj)
    SKW_CUDA(ctx, cudaMemcpyAsync(h_xadj, ctx->xadj, sizeof(uint32_t) * ((size_t)ctx->V + 1),
                                  cudaMemcpyDeviceToHost, ctx->stream));
  if (h_adjncy && ctx->E)
    SKW_CUDA(ctx, cudaMemcpyAsync(h_adjncy, ctx->adjncy, sizeof(uint32_t) * ctx->E,
                                  cudaMemcpyDeviceToHost, ctx->stream));
  if (h_adjwgt && ctx->E) {
    if (!ctx->adjwgt) return fail(ctx, SKW_ERR_STATE, "skw_graph_download: weights were released");
    SKW_CUDA(ctx, cudaMemcpyAsync(h_adjwgt, ctx->adjwgt, sizeof(float) * ctx->E,
                                  cudaMemcpyDeviceToHost, ctx->stream));
  }
  SKW_CUDA(ctx, cudaStreamSynchronize(ctx->stream));
  return SKW_OK;
}

int skw_graph_device_ptrs(const skw_ctx* ctx, const uint32_t** d_xadj, const uint32_t** d_adjncy,
                          const float** d_adjwgt) {
  if (!ctx) return SKW_ERR_ARG;
  if (d_xadj) *d_xadj = ctx->xadj;
  if (d_adjncy) *d_adjncy = ctx->adjncy;
  if (d_adjwgt) *d_adjwgt = ctx->adjwgt;
  return SKW_OK;
}

int skw_graph_free_weights(skw_ctx* ctx) {
  if (!ctx) return SKW_ERR_ARG;
  DeviceGuard g(ctx->device);
  SKW_CUDA(ctx, cudaStreamSynchronize(ctx->stream));
  if (ctx->owns_weights) SKW_CUDA(ctx, cudaFree(ctx->adjwgt));
  ctx->adjwgt = nullptr;
  ctx->owns_weights = false;
  return SKW_OK;
}

// Galois .gr version 1 (include/graph.cuh:164-327 of the reference), ingested on the GPU: the file
// is read in 64 MB pieces into two pinned buffers that alternate, each piece goes to the device while
// the next one is being read, and what the reference does per element on the host happens there --
// 64-bit end offsets narrowed to 32 bits (and checked against numEdge), 32-bit edge data converted to
// float by value; destinations need no conversion and land in place.  No full-size host array exists
// at any time, and the structural checks (offsets non-decreasing, destinations below V) are the
// device pass every upload goes through.
__global__ void __launch_bounds__(256) narrow_offsets_kernel(const uint64_t* __restrict__ ends, size_t n,
                                                             uint64_t num_edge, uint32_t* __restrict__ xadj_from1,
                                                             uint32_t first_node, uint32_t* __restrict__ err) {
  for (size_t i = blockIdx.x * (size_t)blockDim.x + threadIdx.x; i < n; i += (size_t)gridDim.x * blockDim.x) {
    const uint64_t e = ends[i];
    if (e > num_edge) dev_fail(err, DEV_ERR_INDEX, first_node + (uint32_t)i, (uint32_t)(e >> 32), (uint32_t)e);
    xadj_from1[i] = (uint32_t)(e > num_edge ? num_edge : e);
  }
}
__global__ void __launch_bounds__(256) edge_data_to_float_kernel(const uint32_t* __restrict__ raw, size_t n,
                                                                 float* __restrict__ w) {
  for (size_t i = blockIdx.x * (size_t)blockDim.x + threadIdx.x; i < n; i += (size_t)gridDim.x * blockDim.x)
    w[i] = (float)raw[i];
}

namespace {
// Two pinned buffers and two device buffers of kPiece bytes, used alternately: piece k may be read
// from the file while piece k - 1 is still on its way to the device.
struct GrPipe {
  static constexpr size_t kPiece = 64u << 20;
  skw_ctx* ctx;
  unsigned char* h[2] = {nullptr, nullptr};
  unsigned char* d[2] = {nullptr, nullptr};
  cudaEvent_t done[2] = {nullptr, nullptr};
  bool busy[2] = {false, false};
  int cur = 0;
  explicit GrPipe(skw_ctx* c) : ctx(c) {}
  ~GrPipe() {
    cudaStreamSynchronize(ctx->stream);
    for (int i = 0; i < 2; ++i) {
      if (h[i]) cudaFreeHost(h[i]);
      if (d[i]) cudaFree(d[i]);
      if (done[i]) cudaEventDestroy(done[i]);
    }
  }
  int init() {
    for (int i = 0; i < 2; ++i) {
      SKW_CUDA(ctx, cudaMallocHost(&h[i], kPiece));
      SKW_CUDA(ctx, cudaMalloc(&d[i], kPiece));
      SKW_CUDA(ctx, cudaEventCreateWithFlags(&done[i], cudaEventDisableTiming));
    }
    return SKW_OK;
  }
  // The next free pair of buffers (waits until the device is done with its previous piece).
  int next(int* slot) {
    cur ^= 1;
    if (busy[cur]) SKW_CUDA(ctx, cudaEventSynchronize(done[cur]));
    busy[cur] = false;
    *slot = cur;
    return SKW_OK;
  }
  int submitted(int slot) {
    SKW_CUDA(ctx, cudaEventRecord(done[slot], ctx->stream));
    busy[slot] = true;
    return SKW_OK;
  }
};
}  // namespace

int skw_graph_load_gr(skw_ctx* ctx, const char* path, int weight_mode, uint32_t weightrange,
                      uint64_t weight_seed) {
  if (!ctx || !path) return SKW_ERR_ARG;
  FILE* f = fopen(path, "rb");
  if (!f) return fail(ctx, SKW_ERR_IO, "skw_graph_load_gr: cannot open %s", path);
  struct Closer {
    FILE* f;
    ~Closer() { fclose(f); }
  } closer{f};
  uint64_t hdr[4];
  if (fread(hdr, 8, 4, f) != 4) return fail(ctx, SKW_ERR_IO, "%s: short header", path);
  if (hdr[0] != 1) return fail(ctx, SKW_ERR_IO, "%s: unsupported .gr version %llu", path,
                               (unsigned long long)hdr[0]);
  const uint64_t size_edge_ty = hdr[1], num_node = hdr[2], num_edge = hdr[3];
  if (num_node >= 0xFFFFFFFFull || num_edge > 0xFFFFFFFFull)
    return fail(ctx, SKW_ERR_IO, "%s: %llu nodes / %llu edges do not fit 32-bit ids", path,
                (unsigned long long)num_node, (unsigned long long)num_edge);
  if (size_edge_ty != 0 && size_edge_ty != 4)
    return fail(ctx, SKW_ERR_IO, "%s: edge data of %llu bytes is not supported (want 0 or 4)",
                path, (unsigned long long)size_edge_ty);
  if (weight_mode == 0 && size_edge_ty != 4)
    return fail(ctx, SKW_ERR_IO, "%s: file carries no edge data but weights were requested", path);
  DeviceGuard g(ctx->device);
  free_graph(ctx);
  const uint32_t V = (uint32_t)num_node;
  const uint64_t E = num_edge;
  // on any failure below the half-filled arrays are released again
  auto body = [&]() -> int {
    SKW_CUDA(ctx, cudaMalloc(&ctx->xadj, sizeof(uint32_t) * ((size_t)V + 1)));
    SKW_CUDA(ctx, cudaMalloc(&ctx->adjncy, sizeof(uint32_t) * (E ? E : 1)));
    SKW_CUDA(ctx, cudaMalloc(&ctx->adjwgt, sizeof(float) * (E ? E : 1)));
    ctx->owns_graph = ctx->owns_weights = true;
    ctx->V = V;
    ctx->E = E;
    cudaStream_t st = ctx->stream;
    int rc = err_reset(ctx);
    if (rc != SKW_OK) return rc;
    SKW_CUDA(ctx, cudaMemsetAsync(ctx->xadj, 0, sizeof(uint32_t), st));
    GrPipe pipe(ctx);
    if ((rc = pipe.init()) != SKW_OK) return rc;
    const int grid = ctx->sm_count * 4;
    // numNode x u64 end offsets -> xadj[1 ..]
    for (uint64_t i = 0; i < num_node;) {
      const size_t cnt = (size_t)std::min<uint64_t>(num_node - i, GrPipe::kPiece / 8);
      int s;
      if ((rc = pipe.next(&s)) != SKW_OK) return rc;
      if (fread(pipe.h[s], 8, cnt, f) != cnt) return fail(ctx, SKW_ERR_IO, "%s: short offset array", path);
      SKW_CUDA(ctx, cudaMemcpyAsync(pipe.d[s], pipe.h[s], cnt * 8, cudaMemcpyHostToDevice, st));
      narrow_offsets_kernel<<<grid, 256, 0, st>>>(reinterpret_cast<const uint64_t*>(pipe.d[s]), cnt, num_edge,
                                                 ctx->xadj + 1 + i, (uint32_t)i, ctx->d_err);
      SKW_LAUNCHED(ctx);
      if ((rc = pipe.submitted(s)) != SKW_OK) return rc;
      i += cnt;
    }
    // numEdge x u32 destinations -> adjncy, in place
    for (uint64_t i = 0; i < num_edge;) {
      const size_t cnt = (size_t)std::min<uint64_t>(num_edge - i, GrPipe::kPiece / 4);
      int s;
      if ((rc = pipe.next(&s)) != SKW_OK) return rc;
      if (fread(pipe.h[s], 4, cnt, f) != cnt) return fail(ctx, SKW_ERR_IO, "%s: short destination array", path);
      SKW_CUDA(ctx, cudaMemcpyAsync(ctx->adjncy + i, pipe.h[s], cnt * 4, cudaMemcpyHostToDevice, st));
      if ((rc = pipe.submitted(s)) != SKW_OK) return rc;
      i += cnt;
    }
    if (weight_mode == 0) {
      if (num_edge & 1) {
        uint32_t pad;
        if (fread(&pad, 4, 1, f) != 1) return fail(ctx, SKW_ERR_IO, "%s: short padding", path);
      }
      // numEdge x u32 edge data -> float weights
      for (uint64_t i = 0; i < num_edge;) {
        const size_t cnt = (size_t)std::min<uint64_t>(num_edge - i, GrPipe::kPiece / 4);
        int s;
        if ((rc = pipe.next(&s)) != SKW_OK) return rc;
        if (fread(pipe.h[s], 4, cnt, f) != cnt) return fail(ctx, SKW_ERR_IO, "%s: short edge-data array", path);
        SKW_CUDA(ctx, cudaMemcpyAsync(pipe.d[s], pipe.h[s], cnt * 4, cudaMemcpyHostToDevice, st));
        edge_data_to_float_kernel<<<grid, 256, 0, st>>>(reinterpret_cast<const uint32_t*>(pipe.d[s]), cnt,
                                                       ctx->adjwgt + i);
        SKW_LAUNCHED(ctx);
        if ((rc = pipe.submitted(s)) != SKW_OK) return rc;
        i += cnt;
      }
    } else if (weight_mode == 2 && num_edge) {
      // filled after the structure has been checked (the kernel walks the offsets)
    } else if (weight_mode == 3 && num_edge) {
      fill_random_weights_kernel<<<grid, 256, 0, st>>>(ctx->adjwgt, num_edge, weight_seed, (float)weightrange);
      SKW_LAUNCHED(ctx);
    } else if (num_edge) {
      fill_ones_kernel<<<grid, 256, 0, st>>>(ctx->adjwgt, num_edge);
      SKW_LAUNCHED(ctx);
    }
    rc = err_check(ctx, "skw_graph_load_gr");  // an end offset beyond numEdge
    if (rc == SKW_ERR_DEVICE) {
      const std::string why = ctx->err;
      return fail(ctx, SKW_ERR_IO, "%s: an end offset exceeds numEdge -- %s", path, why.c_str());
    }
    if (rc != SKW_OK) return rc;
    return SKW_OK;
  };
  int rc = body();
  if (rc != SKW_OK) {
    const std::string why = ctx->err;
    cudaStreamSynchronize(ctx->stream);
    free_graph(ctx);
    ctx->err = why;
    return rc;
  }
  // offsets non-decreasing and ending at numEdge, destinations below numNode: the device pass every
  // upload goes through (it releases the graph when it refuses it)
  rc = validate_graph(ctx, "skw_graph_load_gr");
  if (rc != SKW_OK) return rc == SKW_ERR_ARG ? fail(ctx, SKW_ERR_IO, "%s", std::string(ctx->err).c_str()) : rc;
  if (weight_mode == 2 && num_edge) {
    fill_degree_weights_kernel<<<ctx->sm_count * 4, 256, 0, ctx->stream>>>(ctx->xadj, ctx->V, ctx->adjwgt);
    SKW_LAUNCHED(ctx);
  }
  if ((rc = finish_graph(ctx)) != SKW_OK) return rc;
  SKW_CUDA(ctx, cudaStreamSynchronize(ctx->stream));
  return SKW_OK;
}

int skw_alias_export(skw_ctx* ctx, float* h_prob, uint32_t* h_alias, uint8_t* h_valid) {
  if (!ctx) return SKW_ERR_ARG;
  if (!ctx->table_ready) return fail(ctx, SKW_ERR_STATE, "skw_alias_export: no table built");
  DeviceGuard g(ctx->device);
  if ((h_prob || h_alias) && ctx->E) {
    const uint64_t chunk = 32u << 20;  // slots per staging round (256 MB of host memory)
    std::vector<Slot> tmp(ctx->E < chunk ? ctx->E : chunk);
    for (uint64_t o = 0; o < ctx->E; o += chunk) {
      const uint64_t cnt = ctx->E - o < chunk ? ctx->E - o : chunk;
      SKW_CUDA(ctx, cudaMemcpyAsync(tmp.data(), ctx->slots + o, sizeof(Slot) * cnt, cudaMemcpyDeviceToHost,
                                    ctx->stream));
      SKW_CUDA(ctx, cudaStreamSynchronize(ctx->stream));
      for (uint64_t i = 0; i < cnt; ++i) {
        if (h_prob) h_prob[o + i] = tmp[i].prob < 0.0f ? 1.0f : tmp[i].prob;  // -1 marks "no usable weight"
        if (h_alias) h_alias[o + i] = tmp[i].alias;
      }
    }
  }
  if (h_valid && ctx->V) {
    SKW_CUDA(ctx, cudaMemcpyAsync(h_valid, ctx->valid, ctx->V, cudaMemcpyDeviceToHost, ctx->stream));
    SKW_CUDA(ctx, cudaStreamSynchronize(ctx->stream));
  }
  return SKW_OK;
}

int skw_alias_import(skw_ctx* ctx, const float* h_prob, const uint32_t* h_alias,
                     const uint8_t* h_valid) {
  if (!ctx) return SKW_ERR_ARG;
  if (!ctx->xadj) return fail(ctx, SKW_ERR_STATE, "skw_alias_import: no graph resident");
  if (!h_prob || !h_alias || !h_valid) return fail(ctx, SKW_ERR_ARG, "skw_alias_import: null array");
  DeviceGuard g(ctx->device);
  drop_records(ctx);
  int rc = alloc_table(ctx);
  if (rc != SKW_OK) return rc;
  std::vector<Slot> tmp(ctx->E ? ctx->E : 1);
  for (uint64_t i = 0; i < ctx->E; ++i) {
    tmp[i].prob = h_prob[i];
    tmp[i].alias = h_alias[i];
  }
  {  // a vertex flagged invalid carries prob = -1 in all of its slots: the draw kernels test that
    std::vector<uint32_t> xadj((size_t)ctx->V + 1);
    SKW_CUDA(ctx, cudaMemcpyAsync(xadj.data(), ctx->xadj, sizeof(uint32_t) * ((size_t)ctx->V + 1),
                                  cudaMemcpyDeviceToHost, ctx->stream));
    SKW_CUDA(ctx, cudaStreamSynchronize(ctx->stream));
    for (uint32_t v = 0; v < ctx->V; ++v)
      if (!h_valid[v])
        for (uint32_t i = xadj[v]; i < xadj[v + 1]; ++i) tmp[i].prob = -1.0f;
  }
  if (ctx->E)
    SKW_CUDA(ctx, cudaMemcpyAsync(ctx->slots, tmp.data(), sizeof(Slot) * ctx->E,
                                  cudaMemcpyHostToDevice, ctx->stream));
  if (ctx->V)
    SKW_CUDA(ctx, cudaMemcpyAsync(ctx->valid, h_valid, ctx->V, cudaMemcpyHostToDevice, ctx->stream));
  SKW_CUDA(ctx, cudaStreamSynchronize(ctx->stream));
  ctx->table_ready = false;
  if ((rc = validate_table(ctx, "skw_alias_import")) != SKW_OK) return rc;
  ctx->table_ready = true;
  return SKW_OK;
}

// Table checkpoint: 48-byte header {magic "SKWTABLE", V, E, slot bytes, fingerprint of the offset
// array, 0} + E packed slots + V valid bytes.  A built table is a pure function of the graph, so a
// checkpoint saves only the build time.
static const char kTableMagic[8] = {'S', 'K', 'W', 'T', 'A', 'B', 'L', 'E'};

int skw_alias_save(skw_ctx* ctx, const char* path) {
  if (!ctx || !path) return SKW_ERR_ARG;
  if (!ctx->table_ready) return fail(ctx, SKW_ERR_STATE, "skw_alias_save: no table built");
  DeviceGuard g(ctx->device);
  FILE* f = fopen(path, "wb");
  if (!f) return fail(ctx, SKW_ERR_IO, "skw_alias_save: cannot create %s", path);
  uint64_t hdr[6];
  memcpy(&hdr[0], kTableMagic, 8);
  hdr[1] = ctx->V;
  hdr[2] = ctx->E;
  hdr[3] = sizeof(Slot);
  hdr[5] = 0;
  if (xadj_fingerprint(ctx, &hdr[4]) != SKW_OK) {
    fclose(f);
    return SKW_ERR_CUDA;
  }
  bool ok = fwrite(hdr, 8, 6, f) == 6;
  const size_t chunk = 64u << 20;  // staged through a bounded host buffer
  std::vector<unsigned char> buf(chunk);
  auto dump = [&](const void* dptr, size_t bytes) {
    for (size_t o = 0; ok && o < bytes; o += chunk) {
      const size_t nb = bytes - o < chunk ? bytes - o : chunk;
      if (cudaMemcpyAsync(buf.data(), static_cast<const unsigned char*>(dptr) + o, nb, cudaMemcpyDeviceToHost,
                          ctx->stream) != cudaSuccess ||
          cudaStreamSynchronize(ctx->stream) != cudaSuccess)
        ok = false;
      else
        ok = fwrite(buf.data(), 1, nb, f) == nb;
    }
  };
  dump(ctx->slots, sizeof(Slot) * ctx->E);
  dump(ctx->valid, ctx->V);
  ok = (fclose(f) == 0) && ok;
  if (!ok) return fail(ctx, SKW_ERR_IO, "skw_alias_save: write to %s failed", path);
  return SKW_OK;
}

int skw_alias_load(skw_ctx* ctx, const char* path) {
  if (!ctx || !path) return SKW_ERR_ARG;
  if (!ctx->xadj) return fail(ctx, SKW_ERR_STATE, "skw_alias_load: no graph resident");
  DeviceGuard g(ctx->device);
  FILE* f = fopen(path, "rb");
  if (!f) return fail(ctx, SKW_ERR_IO, "skw_alias_load: cannot open %s", path);
  struct Closer {
    FILE* f;
    ~Closer() { fclose(f); }
  } closer{f};
  uint64_t hdr[6];
  if (fread(hdr, 8, 6, f) != 6 || memcmp(&hdr[0], kTableMagic, 8) != 0)
    return fail(ctx, SKW_ERR_IO, "skw_alias_load: %s is not a table checkpoint", path);
  if (hdr[1] != ctx->V || hdr[2] != ctx->E || hdr[3] != sizeof(Slot))
    return fail(ctx, SKW_ERR_IO, "skw_alias_load: %s holds a table for V=%llu E=%llu, the resident graph has V=%u E=%llu",
                path, (unsigned long long)hdr[1], (unsigned long long)hdr[2], ctx->V, (unsigned long long)ctx->E);
  uint64_t fp = 0;
  int rc = xadj_fingerprint(ctx, &fp);
  if (rc != SKW_OK) return rc;
  if (hdr[4] != fp)
    return fail(ctx, SKW_ERR_IO, "skw_alias_load: %s was written for another graph (same V and E, different offsets)", path);
  drop_records(ctx);
  rc = alloc_table(ctx);
  if (rc != SKW_OK) return rc;
  ctx->table_ready = false;
  const size_t chunk = 64u << 20;
  std::vector<unsigned char> buf(chunk);
  auto fill = [&](void* dptr, size_t bytes) -> int {
    for (size_t o = 0; o < bytes; o += chunk) {
      const size_t nb = bytes - o < chunk ? bytes - o : chunk;
      if (fread(buf.data(), 1, nb, f) != nb) return fail(ctx, SKW_ERR_IO, "skw_alias_load: %s is truncated", path);
      SKW_CUDA(ctx, cudaMemcpyAsync(static_cast<unsigned char*>(dptr) + o, buf.data(), nb, cudaMemcpyHostToDevice,
                                    ctx->stream));
      SKW_CUDA(ctx, cudaStreamSynchronize(ctx->stream));
    }
    return SKW_OK;
  };
  if ((rc = fill(ctx->slots, sizeof(Slot) * ctx->E)) != SKW_OK) return rc;
  if ((rc = fill(ctx->valid, ctx->V)) != SKW_OK) return rc;
  if ((rc = validate_table(ctx, "skw_alias_load")) != SKW_OK) return rc;
  ctx->table_ready = true;
  return SKW_OK;
}

int skw_alias_device_ptrs(const skw_ctx* ctx, const void** d_slots, const uint8_t** d_valid) {
  if (!ctx) return SKW_ERR_ARG;
  if (d_slots) *d_slots = ctx->slots;
  if (d_valid) *d_valid = ctx->valid;
  return SKW_OK;
}

int skw_host_alloc(size_t bytes, void** out) {
  if (!out) return SKW_ERR_ARG;
  cudaError_t e = cudaMallocHost(out, bytes ? bytes : 1);
  if (e != cudaSuccess) {
    *out = nullptr;
    return fail(nullptr, SKW_ERR_NOMEM, "skw_host_alloc(%zu): %s", bytes, cudaGetErrorString(e));
  }
  return SKW_OK;
}

void skw_host_free(void* p) {
  if (p) cudaFreeHost(p);
}

}  // extern "C"
