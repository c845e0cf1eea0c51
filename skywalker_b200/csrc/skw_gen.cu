// Seeded synthetic graphs generated on the GPU: R-MAT and a capped power-law graph, plus the
// per-edge weights.  These stand in for the datasets the reference's scripts use
// (scripts/fig8_biased.sh:9-24: web-Google ... Friendster), none of which ship with it.
// Input preparation only: sorting and compaction use CUB; nothing here is on the sampling path.
#include <cmath>
#include <cub/cub.cuh>
#include <vector>

#include "skw_ctx.h"

namespace skw {

__device__ __forceinline__ u32 scramble(u32 v, u32 scale) {
  const u32 mask = scale >= 32 ? 0xFFFFFFFFu : ((1u << scale) - 1u);
  const u32 sh = scale / 2 ? scale / 2 : 1;
  v = (v * 0x9E3779B1u) & mask;
  v ^= v >> sh;
  v = (v * 0x85EBCA6Bu) & mask;
  v ^= v >> sh;
  return v;
}

// One raw edge per thread: `scale` quadrant choices, one Philox word each.
__global__ void __launch_bounds__(256) rmat_keys_kernel(u64* __restrict__ keys, u64 raw_edges,
                                                        u32 scale, u32 ta, u32 tab, u32 tabc,
                                                        int symmetric, u64 seed, u64 sentinel,
                                                        u32 fold) {
  for (u64 e = (u64)blockIdx.x * blockDim.x + threadIdx.x; e < raw_edges; e += (u64)gridDim.x * blockDim.x) {
    u32 src = 0, dst = 0;
    Rand4 r{0, 0, 0, 0};
    for (u32 l = 0; l < scale; ++l) {
      if ((l & 3) == 0) r = philox_tagged(seed, TAG_RMAT, e, l >> 2, 0);
      const u32 x = (l & 3) == 0 ? r.x : (l & 3) == 1 ? r.y : (l & 3) == 2 ? r.z : r.w;
      const u32 sb = x >= tab ? 1u : 0u;
      const u32 db = ((x >= ta && x < tab) || x >= tabc) ? 1u : 0u;
      src = (src << 1) | sb;
      dst = (dst << 1) | db;
    }
    src = scramble(src, scale);
    dst = scramble(dst, scale);
    if (fold) {
      src %= fold;
      dst %= fold;
    }
    const bool loop = src == dst;
    if (symmetric) {
      keys[2 * e] = loop ? sentinel : (((u64)src << 32) | dst);
      keys[2 * e + 1] = loop ? sentinel : (((u64)dst << 32) | src);
    } else {
      keys[e] = loop ? sentinel : (((u64)src << 32) | dst);
    }
  }
}

__device__ __forceinline__ u32 upper_bound_vertex(const u64* __restrict__ cum, u32 V, u64 x) {
  u32 lo = 0, hi = V + 1;  // first index with cum[i] > x
  while (lo < hi) {
    const u32 mid = lo + ((hi - lo) >> 1);
    if (cum[mid] <= x) lo = mid + 1;
    else hi = mid;
  }
  return lo - 1;
}

__global__ void __launch_bounds__(256) powerlaw_keys_kernel(u64* __restrict__ keys, u64 raw_edges,
                                                            const u64* __restrict__ cum, u32 V,
                                                            u64 seed, u64 sentinel) {
  const u64 S = cum[V];
  for (u64 e = (u64)blockIdx.x * blockDim.x + threadIdx.x; e < raw_edges; e += (u64)gridDim.x * blockDim.x) {
    const Rand4 r = philox_tagged(seed, TAG_PLAW, e, 0, 0);
    const u64 x = __umul64hi(((u64)r.x << 32) | r.y, S);
    const u64 y = __umul64hi(((u64)r.z << 32) | r.w, S);
    const u32 a = upper_bound_vertex(cum, V, x);
    const u32 b = upper_bound_vertex(cum, V, y);
    keys[2 * e] = a == b ? sentinel : (((u64)a << 32) | b);
    keys[2 * e + 1] = a == b ? sentinel : (((u64)b << 32) | a);
  }
}

// keys sorted and unique, E of them: adjncy[i] = low word; xadj[v] = first i whose source >= v.
__global__ void __launch_bounds__(256) csr_from_keys_kernel(const u64* __restrict__ keys, u64 E,
                                                            u32 V, u32* __restrict__ xadj,
                                                            u32* __restrict__ adjncy) {
  for (u64 i = (u64)blockIdx.x * blockDim.x + threadIdx.x; i <= E; i += (u64)gridDim.x * blockDim.x) {
    const u32 src = i < E ? (u32)(keys[i] >> 32) : V;
    const u32 before = i ? (u32)(keys[i - 1] >> 32) + 1 : 0;
    for (u32 v = before; v <= src; ++v) xadj[v] = (u32)i;
    if (i < E) adjncy[i] = (u32)keys[i];
  }
}

__global__ void __launch_bounds__(256) edge_weights_kernel(float* __restrict__ w, u64 E, u64 seed) {
  for (u64 e = (u64)blockIdx.x * blockDim.x + threadIdx.x; e < E; e += (u64)gridDim.x * blockDim.x) {
    const Rand4 r = philox_tagged(seed, TAG_WGHT, e, 0, 0);
    const u32 val = (1u << 20) + (((r.x >> 8) * 9u) >> 4);
    w[e] = (float)val * 9.5367431640625e-7f;
  }
}

// keys (count of them, device) -> sorted unique CSR resident in ctx.
static int keys_to_graph(skw_ctx* ctx, u64* keys, u64* alt, u64 count, u32 V, int key_bits,
                         u64 sentinel, u64 weight_seed) {
  cudaStream_t st = ctx->stream;
  void* tmp = nullptr;
  size_t tmp_bytes = 0, need = 0;
  cub::DoubleBuffer<u64> buf(keys, alt);
  cub::DeviceRadixSort::SortKeys(nullptr, need, buf, (long long)count, 0, key_bits, st);
  tmp_bytes = need;
  u64* d_num = nullptr;
  size_t need2 = 0;
  cub::DeviceSelect::Unique(nullptr, need2, keys, alt, d_num, (long long)count, st);
  if (need2 > tmp_bytes) tmp_bytes = need2;
  SKW_CUDA(ctx, cudaMalloc(&tmp, tmp_bytes + 16));
  struct Free {
    void* p;
    ~Free() { cudaFree(p); }
  } f1{tmp};
  SKW_CUDA(ctx, cudaMalloc(&d_num, sizeof(u64)));
  Free f2{d_num};
  need = tmp_bytes;
  SKW_CUDA(ctx, cub::DeviceRadixSort::SortKeys(tmp, need, buf, (long long)count, 0, key_bits, st));
  ctx->launches += 8;  // library kernels, counted roughly
  u64* sorted = buf.Current();
  u64* out = buf.Alternate();
  need2 = tmp_bytes;
  SKW_CUDA(ctx, cub::DeviceSelect::Unique(tmp, need2, sorted, out, d_num, (long long)count, st));
  u64 h_num = 0;
  SKW_CUDA(ctx, cudaMemcpyAsync(&h_num, d_num, sizeof(u64), cudaMemcpyDeviceToHost, st));
  SKW_CUDA(ctx, cudaStreamSynchronize(st));
  u64 E = h_num;
  if (E) {
    u64 last = 0;
    SKW_CUDA(ctx, cudaMemcpy(&last, out + (E - 1), sizeof(u64), cudaMemcpyDeviceToHost));
    if (last == sentinel) --E;
  }
  if (E > 0xFFFFFFFFull) return fail(ctx, SKW_ERR_ARG, "generated graph has %llu edges: more than 32-bit offsets hold",
                                     (unsigned long long)E);
  u32 *xadj = nullptr, *adjncy = nullptr;
  float* wgt = nullptr;
  SKW_CUDA(ctx, cudaMalloc(&xadj, sizeof(u32) * ((size_t)V + 1)));
  SKW_CUDA(ctx, cudaMalloc(&adjncy, sizeof(u32) * (E ? E : 1)));
  SKW_CUDA(ctx, cudaMalloc(&wgt, sizeof(float) * (E ? E : 1)));
  const int grid = ctx->sm_count * 8;
  csr_from_keys_kernel<<<grid, 256, 0, st>>>(out, E, V, xadj, adjncy);
  SKW_LAUNCHED(ctx);
  edge_weights_kernel<<<grid, 256, 0, st>>>(wgt, E, weight_seed);
  SKW_LAUNCHED(ctx);
  SKW_CUDA(ctx, cudaStreamSynchronize(st));
  int rc = skw_graph_adopt_device(ctx, V, E, xadj, adjncy, wgt);
  if (rc != SKW_OK) {
    cudaFree(xadj);
    cudaFree(adjncy);
    cudaFree(wgt);
    return rc;
  }
  ctx->owns_graph = true;
  ctx->owns_weights = true;
  return SKW_OK;
}

}  // namespace skw

using namespace skw;

extern "C" {

int skw_graph_generate_rmat(skw_ctx* ctx, uint32_t scale, uint32_t num_vertices, uint64_t raw_edges,
                            double a, double b, double c, int symmetric, uint64_t graph_seed,
                            uint64_t weight_seed) {
  if (!ctx) return SKW_ERR_ARG;
  if (scale < 1 || scale > 31) return fail(ctx, SKW_ERR_ARG, "skw_graph_generate_rmat: scale must be 1..31");
  if (!(a >= 0 && b >= 0 && c >= 0 && a + b + c <= 1.0))
    return fail(ctx, SKW_ERR_ARG, "skw_graph_generate_rmat: need a,b,c >= 0 and a+b+c <= 1");
  if (num_vertices > (1u << scale) || num_vertices == 1)
    return fail(ctx, SKW_ERR_ARG, "skw_graph_generate_rmat: num_vertices must be 0 or in 2..2^scale");
  const u32 fold = (num_vertices && num_vertices < (1u << scale)) ? num_vertices : 0;
  DeviceGuard g(ctx->device);
  const u32 ta = (u32)fmin(4294967295.0, a * 4294967296.0);
  const u32 tab = (u32)fmin(4294967295.0, (a + b) * 4294967296.0);
  const u32 tabc = (u32)fmin(4294967295.0, (a + b + c) * 4294967296.0);
  const u64 count = raw_edges * (symmetric ? 2 : 1);
  const u64 sentinel = (u64)1 << (32 + scale);  // a source id one past the last vertex
  u64 *keys = nullptr, *alt = nullptr;
  SKW_CUDA(ctx, cudaMalloc(&keys, sizeof(u64) * (count ? count : 1)));
  SKW_CUDA(ctx, cudaMalloc(&alt, sizeof(u64) * (count ? count : 1)));
  if (raw_edges) {
    rmat_keys_kernel<<<ctx->sm_count * 8, 256, 0, ctx->stream>>>(keys, raw_edges, scale, ta, tab, tabc,
                                                                 symmetric, graph_seed, sentinel, fold);
    ctx->launches++;
  }
  int rc = keys_to_graph(ctx, keys, alt, count, fold ? fold : 1u << scale, 33 + (int)scale, sentinel, weight_seed);
  cudaFree(keys);
  cudaFree(alt);
  return rc;
}

int skw_graph_generate_powerlaw(skw_ctx* ctx, uint32_t V, uint64_t raw_edges, double exponent,
                                double dmin, uint32_t cap, uint64_t graph_seed, uint64_t weight_seed) {
  if (!ctx) return SKW_ERR_ARG;
  if (V < 2 || V >= 0x80000000u) return fail(ctx, SKW_ERR_ARG, "skw_graph_generate_powerlaw: V out of range");
  if (!(exponent > 1.0) || !(dmin > 0.0) || cap < 1)
    return fail(ctx, SKW_ERR_ARG, "skw_graph_generate_powerlaw: need exponent > 1, dmin > 0, cap >= 1");
  DeviceGuard g(ctx->device);
  // target degrees on the host: pow() of the C library, one call per vertex
  std::vector<u64> cum((size_t)V + 1);
  cum[0] = 0;
  const double ex = -1.0 / (exponent - 1.0);
  for (u32 v = 0; v < V; ++v) {
    // same Philox words as the device would draw: counter (v, 0, 0, 1), key seed ^ TAG_PLAW
    u32 c0 = v, c1 = 0, c2 = 0, c3 = 1, k0 = (u32)graph_seed, k1 = (u32)(graph_seed >> 32) ^ TAG_PLAW;
    for (int r = 0; r < 10; ++r) {
      const u64 p0 = (u64)0xD2511F53u * c0, p1 = (u64)0xCD9E8D57u * c2;
      const u32 n0 = (u32)(p1 >> 32) ^ c1 ^ k0, n1 = (u32)p1, n2 = (u32)(p0 >> 32) ^ c3 ^ k1, n3 = (u32)p0;
      c0 = n0; c1 = n1; c2 = n2; c3 = n3;
      k0 += 0x9E3779B9u;
      k1 += 0xBB67AE85u;
    }
    const double u = ((double)(c0 >> 8) + 1.0) * 5.9604644775390625e-8;
    double d = std::floor(dmin * std::pow(u, ex));
    if (!(d < (double)cap)) d = (double)cap;
    if (d < 1.0) d = 1.0;
    cum[v + 1] = cum[v] + (u64)d;
  }
  u64* d_cum = nullptr;
  SKW_CUDA(ctx, cudaMalloc(&d_cum, sizeof(u64) * ((size_t)V + 1)));
  SKW_CUDA(ctx, cudaMemcpyAsync(d_cum, cum.data(), sizeof(u64) * ((size_t)V + 1), cudaMemcpyHostToDevice, ctx->stream));
  const u64 count = raw_edges * 2;
  int bits = 0;
  while (((u64)1 << bits) <= V) ++bits;  // bits of the largest id, and of V itself for the sentinel
  const u64 sentinel = (u64)V << 32;
  u64 *keys = nullptr, *alt = nullptr;
  SKW_CUDA(ctx, cudaMalloc(&keys, sizeof(u64) * (count ? count : 1)));
  SKW_CUDA(ctx, cudaMalloc(&alt, sizeof(u64) * (count ? count : 1)));
  if (raw_edges) {
    powerlaw_keys_kernel<<<ctx->sm_count * 8, 256, 0, ctx->stream>>>(keys, raw_edges, d_cum, V, graph_seed, sentinel);
    ctx->launches++;
  }
  int rc = keys_to_graph(ctx, keys, alt, count, V, 32 + bits, sentinel, weight_seed);
  cudaFree(keys);
  cudaFree(alt);
  cudaFree(d_cum);
  return rc;
}

}  // extern "C"
