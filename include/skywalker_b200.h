/*
 * skywalker_b200 -- C ABI of the B200-native alias-method sampling / random-walk engine.
 *
 * The reference (wpybtw/Skywalker) is a single CUDA executable with no FFI layer; its
 * "operator interface" is a set of host entry functions called by src/main.cu, each taking a
 * C++ owner object (Sampler / Walker) and returning kernel seconds.  This header is the plain-C
 * boundary a maintainer binds instead: every entry point below names the reference function or
 * type (file:line, paths relative to the reference tree) whose job it takes over.
 *
 * Conventions
 *   - every function returns SKW_OK (0) or a negative skw_status; it never calls exit();
 *     skw_last_error(ctx) gives the text of the last failure on that context.
 *   - one skw_ctx per GPU, used by one host thread at a time (the reference runs one OpenMP
 *     thread per GPU, src/main.cu:252-270).
 *   - pointers named h_* are host memory (pageable or pinned), d_* are device memory of the
 *     context's GPU.  The library never keeps a caller pointer after the call returns, except
 *     the CSR arrays handed over with skw_graph_adopt_device().
 *   - vertex ids, edge offsets and degrees are uint32_t (reference: vtx_t/edge_t,
 *     include/graph.cuh:40-45); weights are float.
 *   - all randomness is Philox4x32-10, counter = (unit id low, unit id high, step, trial),
 *     key = 64-bit seed xor a per-purpose tag.  Results therefore do not depend on launch
 *     shape, on the number of GPUs, or on how units are split between calls.
 *   - there is no CPU fallback: without a CUDA device every compute entry point fails with
 *     SKW_ERR_CUDA.
 */
#ifndef SKYWALKER_B200_H
#define SKYWALKER_B200_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

typedef struct skw_ctx skw_ctx;

typedef enum skw_status {
  SKW_OK = 0,
  SKW_ERR_ARG = -1,      /* bad argument (null pointer, size out of range, wrong state) */
  SKW_ERR_CUDA = -2,     /* a CUDA runtime call failed; text in skw_last_error           */
  SKW_ERR_STATE = -3,    /* call order wrong (no graph, no table ...)                    */
  SKW_ERR_DEVICE = -4,   /* a kernel reported an internal error word (bounded wait ran  *
                          * out, index out of range, capacity exceeded)                  */
  SKW_ERR_IO = -5,       /* file could not be read / malformed .gr                       */
  SKW_ERR_NOMEM = -6
} skw_status;

/* walk applications (reference presets: src/main.cu:156-175) */
typedef enum skw_app {
  SKW_APP_DEEPWALK = 0,  /* fixed length, no termination                                   */
  SKW_APP_PPR = 1,       /* before every step stop with probability tp                      *
                          * (reference rule: src/online_walk.cu:109-125, unbiased_walk.cu:82) */
  SKW_APP_NODE2VEC = 2   /* 2nd-order walk, rejection against max(1/p,1,1/q)                *
                          * (reference: src/api/bias_node2vec.cu:14-24, unbiased_walk.cu:14-61) */
} skw_app;

/* where the alias table of the current vertex comes from (reference flag --ol) */
typedef enum skw_mode {
  SKW_MODE_OFFLINE = 0,  /* prebuilt table of all vertices (skw_alias_build_offline)        */
  SKW_MODE_ONLINE = 1    /* table built on the fly for the vertex being left, then dropped  */
} skw_mode;

/* k-hop flags */
#define SKW_KHOP_TAKE_ALL 1u /* reference behaviour (src/offline_sample.cu:120-128): when the  *
                              * fan-out is >= degree copy every neighbour instead of drawing  */

#define SKW_KHOP_UNBIASED 2u /* uniform draws with replacement, no table (--bias=0,            *
                              * src/unbiased_sample.cu:28-36); `mode` is ignored               */

#define SKW_KHOP_DISTINCT 4u /* the rule of the reference's ONLINE sampler (roll_atomic / roll_once,   *
                             * src/online_sample_new.cu:73-111, 3-37): a vertex whose degree is <=   *
                             * the fan-out hands over every neighbour once; otherwise a draw counts  *
                             * only if its column was not drawn before, for at most 352 numbered     *
                             * trials (32 lanes x 11 rounds there); sample_lengths holds how many    *
                             * distinct neighbours were found.  Fan-outs up to 256.  Ignored with    *
                             * SKW_KHOP_UNBIASED.                                                    */

#define SKW_INVALID_VERTEX 0xFFFFFFFFu /* written into k-hop cells that hold no sample */

/* ---------------------------------------------------------------- context ---------------- */

/* Replaces the per-thread cudaSetDevice/cudaFree(0) set-up of src/main.cu:268-270. */
int skw_ctx_create(int device, skw_ctx** out);
void skw_ctx_destroy(skw_ctx* ctx);
const char* skw_last_error(const skw_ctx* ctx);
/* Library-wide text of the last failure of a call that had no context (skw_ctx_create). */
const char* skw_last_global_error(void);
/* All later work of ctx is issued on `cuda_stream` (a cudaStream_t; NULL = the context's own
 * stream).  Lets a caller time the kernels with its own events. */
int skw_ctx_set_stream(skw_ctx* ctx, void* cuda_stream);
int skw_ctx_synchronize(skw_ctx* ctx);
/* Number of kernels of this library launched by ctx since creation. */
uint64_t skw_ctx_kernel_launches(const skw_ctx* ctx);

/* ---------------------------------------------------------------- graph ------------------ */

/* Copy a host CSR to the GPU.  Replaces gpu_graph::gpu_graph (include/gpu_graph.cuh:68-117)
 * in its --gmgraph placement.  xadj has V+1 entries (xadj[0] == 0, xadj[V] == E); adjwgt may
 * be NULL (all weights 1).  Adjacency lists must be sorted ascending for node2vec. */
int skw_graph_upload(skw_ctx* ctx, uint32_t V, uint64_t E, const uint32_t* h_xadj,
                     const uint32_t* h_adjncy, const float* h_adjwgt);
/* Use CSR arrays that already live on the GPU (borrowed until the context is destroyed or
 * another graph is set). */
int skw_graph_adopt_device(skw_ctx* ctx, uint32_t V, uint64_t E, const uint32_t* d_xadj,
                           const uint32_t* d_adjncy, const float* d_adjwgt);
/* Read a Galois .gr (version 1) file and upload it.  Replaces Graph::ReadGraphGR
 * (include/graph.cuh:164-327): header 4 x u64 {1, sizeEdgeTy, numNode, numEdge}, numNode x u64
 * end offsets, numEdge x u32 destinations, 4-byte pad when numEdge is odd, numEdge x u32 edge
 * data converted to float by value.  weight_mode: 0 = from file (--weight), 1 = all ones,
 * 2 = out-degree of the source (--dw), 3 = seeded uniform in [0, weightrange)
 * (--randomweight). */
int skw_graph_load_gr(skw_ctx* ctx, const char* path, int weight_mode, uint32_t weightrange,
                      uint64_t weight_seed);
int skw_graph_info(const skw_ctx* ctx, uint32_t* V, uint64_t* E, uint32_t* max_degree);
/* Copy the resident CSR back to the host (any pointer may be NULL). */
int skw_graph_download(skw_ctx* ctx, uint32_t* h_xadj, uint32_t* h_adjncy, float* h_adjwgt);
/* Device addresses of the resident CSR (for callers that keep everything on the GPU). */
int skw_graph_device_ptrs(const skw_ctx* ctx, const uint32_t** d_xadj,
                          const uint32_t** d_adjncy, const float** d_adjwgt);
/* Release the weights after an offline build, as src/createTable.cu:175-177 does. */
int skw_graph_free_weights(skw_ctx* ctx);

/* Seeded synthetic graphs, generated on the GPU (stand-ins for the datasets of
 * scripts/fig8_biased.sh:9-24).  R-MAT: 2^scale vertices, raw_edges draws with quadrant
 * probabilities (a,b,c,1-a-b-c), ids scrambled by a fixed bijection (then taken modulo
 * num_vertices when 0 < num_vertices < 2^scale, for vertex counts that are not powers of two),
 * duplicates and self loops removed, adjacency sorted; symmetric != 0 adds every reverse edge.  Weights are
 * 1 + 9 * k / 2^24 rounded down to a multiple of 2^-20, k a 24-bit Philox draw per edge. */
int skw_graph_generate_rmat(skw_ctx* ctx, uint32_t scale, uint32_t num_vertices, uint64_t raw_edges,
                            double a, double b, double c, int symmetric, uint64_t graph_seed,
                            uint64_t weight_seed);
/* Power-law graph: vertex v gets target degree min(cap, floor(dmin * u^(-1/(exponent-1)))),
 * endpoints of raw_edges undirected edges are drawn proportionally to target degree, the edge
 * set is symmetrised, de-duplicated, self loops dropped, adjacency sorted. */
int skw_graph_generate_powerlaw(skw_ctx* ctx, uint32_t V, uint64_t raw_edges, double exponent,
                                double dmin, uint32_t cap, uint64_t graph_seed,
                                uint64_t weight_seed);
/* start[i] = mulhi32(philox(seed; id_base + i).x, V): uniformly random start vertices. */
int skw_generate_starts_device(skw_ctx* ctx, uint64_t n, uint64_t id_base, uint64_t seed,
                               uint32_t* d_starts);

/* ---------------------------------------------------------------- alias table ------------ */

/* Build the alias table of vertices [v_begin, v_end) from the resident weights.  Replaces
 * ConstructTable (src/createTable.cu:119-179) and, inside it, loadFromGraph / construct /
 * constructBC / SaveAliasTable of include/alias_table_new.cuh (1077-1132, 1211-1316, 334-464,
 * 1105-1115).  The table of a vertex is a pure function of its weight list (see
 * skw_alias_vertex_spec below), so the result does not depend on scheduling.  *ms receives the
 * build kernels' time (may be NULL). */
int skw_alias_build_offline(skw_ctx* ctx, uint32_t v_begin, uint32_t v_end, float* ms);
/* Copy the table out / in as the reference's two arrays (gpu_graph::prob_array, alias_array,
 * valid; include/gpu_graph.cuh:40-60): prob[E] float, alias[E] uint32 (index inside the
 * vertex's list), valid[V] bytes.  Any pointer may be NULL. */
int skw_alias_export(skw_ctx* ctx, float* h_prob, uint32_t* h_alias, uint8_t* h_valid);
int skw_alias_import(skw_ctx* ctx, const float* h_prob, const uint32_t* h_alias,
                     const uint8_t* h_valid);
/* Checkpoint of the built table in a file (the reference only has the in-process --built flag,
 * src/main.cu:347).  Loading checks that the file was written for a graph of the same V and E. */
int skw_alias_save(skw_ctx* ctx, const char* path);
int skw_alias_load(skw_ctx* ctx, const char* path);
/* Device address of the packed table: E slots of {float prob; uint32 alias} and V valid bytes.  The
 * slot array is allocated with 1024 spare entries past E, so that ranks of a multi-GPU job can
 * all-gather it in place in equal chunks of ceil(E / ranks) slots. */
int skw_alias_device_ptrs(const skw_ctx* ctx, const void** d_slots, const uint8_t** d_valid);

/* Alias table of ONE weight list without any allocation.  No counterpart in the reference (its
 * builders cudaMalloc their scratch per launch, src/createTable.cu:143-159); added for hosts that
 * cannot allocate device memory when they call: a plug-in inside a process whose framework took
 * all HBM for its own pool at start-up, or a serving loop that cannot take the device-wide
 * synchronisation of cudaMalloc / cudaFree on its request path.
 *   d_weights[n]  device, float    the weight list (same rules as an adjacency list's weights)
 *   d_slots[n]    device, 8 bytes each, 8-byte aligned: {float prob; uint32 alias}; prob = -1 in
 *                 every slot when no weight is usable
 *   d_valid[1]    device, 1 if the list has a usable weight, else 0
 *   cuda_stream   a cudaStream_t (NULL = legacy default stream); the call returns after the
 *                 stream has finished the build
 *   errbuf        optional caller buffer that receives the text of a failure
 * All buffers belong to the caller and to the CURRENT device of the calling thread.  n must be
 * 1 .. 131072: the prefix arrays (20 bytes per weight) live in a 2.5 MiB array inside the library
 * image, present on every GPU that loads the library until the process exits; longer lists are
 * rejected with SKW_ERR_ARG.  The result is bit-identical to what skw_alias_build_offline writes
 * for a vertex with this weight list.
 * The first call on a device looks up the array's device address (and, where the CUDA runtime
 * loads modules lazily, is what places the array and the kernel on the GPU): make it at start-up,
 * before the host's own pool reserves the remaining memory, and outside any stream capture.  The
 * address is remembered per device for the life of the process and does not survive a
 * cudaDeviceReset() by the host.  Every call uses the same array, which keeps whatever the previous call
 * left (the call clears the part that must start at zero): two calls whose kernels can overlap
 * on the GPU (different streams, different threads) race on it and must be serialised by the
 * caller.  The function calls no cudaMalloc / cudaFree and no allocating library routine. */
int skw_alias_build_list_static(const float* d_weights, uint32_t n, void* d_slots, uint8_t* d_valid,
                                void* cuda_stream, char* errbuf, size_t errbuf_len);

/* ---------------------------------------------------------------- walks ------------------ */

/* Parameters shared by the walk entry points.  hop_num = walk length + 1 (reference
 * Jobs_result<RW>::hop_num, include/sampler_result.cuh:459). */
typedef struct skw_walk_params {
  uint32_t app;         /* skw_app                                                     */
  uint32_t mode;        /* skw_mode                                                    */
  uint32_t hop_num;     /* cells per path row = max steps + 1                          */
  float tp;             /* PPR termination probability (ignored unless app == PPR)     */
  float p, q;           /* node2vec hyper-parameters                                   */
  uint64_t seed;        /* Philox seed                                                 */
  uint64_t walker_base; /* global id of walker 0 of this call (multi-GPU sharding)     */
  uint64_t walker_stride; /* global id of walker i = walker_base + i * walker_stride; 0 means 1. *
                           * The reference interleaves walkers over GPUs (id = dev + i * ngpu,  *
                           * include/sampler.cuh:494-503): stride = ngpu reproduces that.         */
  uint32_t flags;         /* SKW_WALK_* */
} skw_walk_params;

/* Online walks: keep the table of a vertex for the rest of the call once it has been built, instead
 * of rebuilding the frontier's tables at every step (the reference's --cache flag, src/main.cu:74).
 * The walks are identical; only the amount of build work changes. */
#define SKW_WALK_CACHE_TABLES 1u
/* Unbiased walk (the reference's --bias=0, src/unbiased_walk.cu:102-124): the neighbour is drawn
 * uniformly, no alias table is read or built and `mode` is ignored; with SKW_APP_NODE2VEC this is
 * the reference's unweighted rejection walk (src/unbiased_walk.cu:14-61). */
#define SKW_WALK_UNBIASED 2u
/* Online mode only: how the slot a walker draws is obtained.  BUILD_TABLES: the alias tables of all
 * distinct frontier vertices are built at every step, as OnlineWalkShMem does
 * (src/online_walk.cu:82-166), and the walkers draw from them.  DIRECT_SLOTS: every walker computes
 * the one slot it draws straight from the weight list of its vertex (one warp per walker, all steps
 * in one launch, no table memory touched) -- the same (prob, alias) bits a built table holds, so
 * the walks are identical.  With neither flag the library computes slots directly (for the duration
 * of a call it memoises, per vertex, the largest weight, the total and prefix sums at every 64th list
 * position -- never a table entry).  SKW_WALK_CACHE_TABLES implies BUILD_TABLES. */
#define SKW_WALK_BUILD_TABLES 4u
#define SKW_WALK_DIRECT_SLOTS 8u

/* Optional wider layout of the same table for offline DeepWalk / PPR.  No counterpart in the
 * reference (whose step reads xadj, prob_array, alias_array and adjncy separately,
 * src/offline_walk.cu:89-112).  Derives from the alias table one 32-byte record per edge slot
 * {prob, neighbour-if-kept, its offset, its usable degree, neighbour-via-alias, its offset, its
 * usable degree, alias} (32 B x E of device memory, plus 8 B x V), so that a step is a single
 * random 32-byte access.  Once built, skw_walk* use it for offline DeepWalk and PPR; walks are
 * bit-identical with and without it.  Must be rebuilt after the table changes. */
int skw_walk_records_build(skw_ctx* ctx, float* ms);
int skw_walk_records_free(skw_ctx* ctx);

/* Run n walkers.  Replaces OfflineWalk (src/offline_walk.cu:181-230) for mode OFFLINE and
 * OnlineWalkShMem / OnlineWalkGMem (src/online_walk.cu:245-327, src/online_walk_gmem.cu) for
 * mode ONLINE.  Output layout is Jobs_result<RW> (include/sampler_result.cuh:607-612):
 * paths[w * hop_num + s] = vertex after s steps (s = 0 is the start), lengths[w] = number of
 * steps taken (= sampled edges of that walker; hop_num - 1 unless the walk met a vertex with
 * no usable out-edge or PPR stopped it).  Cells after paths[w * hop_num + lengths[w]] are not
 * written.  *ms = kernel time, *sampled_edges = sum of lengths (both may be NULL). */
int skw_walk_device(skw_ctx* ctx, const skw_walk_params* prm, const uint32_t* d_starts,
                    uint64_t n, uint32_t* d_paths, uint32_t* d_lengths, float* ms,
                    uint64_t* sampled_edges);
/* Enqueue-only form: when ms and sampled_edges are both NULL, skw_walk_device returns as soon as
 * the kernels are queued on the context's stream (no synchronisation, no readback), so back to
 * back calls leave no host gap between kernels.  The sampled edges of such calls add up in the
 * context; skw_ctx_take_sampled_edges() waits for the stream, reports a device error of any of
 * them, returns the sum and clears it. */
int skw_ctx_take_sampled_edges(skw_ctx* ctx, uint64_t* out);
/* Same with host buffers: copies starts in, runs, copies paths and lengths out.  When h_paths is
 * pinned memory (skw_host_alloc, cudaHostAlloc, cudaHostRegister) only the cells each walk wrote
 * (0 .. length) are transferred, by a kernel writing into the mapped host matrix; the other cells
 * keep what the caller had there.  With pageable memory the whole matrix is copied and cells past a
 * walk's end are unspecified. */
int skw_walk(skw_ctx* ctx, const skw_walk_params* prm, const uint32_t* h_starts, uint64_t n,
             uint32_t* h_paths, uint32_t* h_lengths, float* ms, uint64_t* sampled_edges);
/* Host buffers, packed result.  No counterpart in the reference, which leaves results on the
 * device (include/sampler_result.cuh:571-612).  h_lengths[w] as in skw_walk; h_packed receives the
 * walks back to back in walker order, walk w holding lengths[w] + 1 vertices (its start first)
 * from cell sum_{u<w}(lengths[u] + 1) on -- the same values the row layout holds in
 * paths[w * hop_num + 0 .. lengths[w]].  *cells = cells the result needs (= sampled edges + n).
 * When capacity_cells is smaller (or h_packed is NULL) the call fills h_lengths and *cells, leaves
 * h_packed unspecified (never written past capacity_cells) and returns SKW_ERR_ARG; the same call
 * with a buffer of *cells cells then returns the same walks.  Rows are packed on the device and
 * leave in contiguous copies, so only cells that hold a result cross the bus; large batches run as
 * a pipeline of slices whose copies overlap the next slice's walk (fastest with pinned buffers). */
int skw_walk_packed(skw_ctx* ctx, const skw_walk_params* prm, const uint32_t* h_starts, uint64_t n,
                    uint32_t* h_packed, uint64_t capacity_cells, uint32_t* h_lengths, uint64_t* cells,
                    float* ms, uint64_t* sampled_edges);
/* The same with one byte per length (h_lengths8[w] = lengths[w]); prm->hop_num must not exceed 256,
 * so that every length fits.  The lengths are a sixth of what a PPR batch sends home (about 2.6
 * vertices per walk at tp = 0.15), and the result is bound by the bus. */
int skw_walk_packed_u8(skw_ctx* ctx, const skw_walk_params* prm, const uint32_t* h_starts, uint64_t n,
                       uint32_t* h_packed, uint64_t capacity_cells, uint8_t* h_lengths8, uint64_t* cells,
                       float* ms, uint64_t* sampled_edges);

/* ---------------------------------------------------------------- k-hop sampling --------- */

typedef struct skw_khop_params {
  uint32_t mode;        /* skw_mode                                                    */
  uint32_t nhops;       /* number of hops (reference --d), 1..4                         */
  uint32_t fanout[4];   /* samples per vertex at hop 1..nhops (reference hops[1..])     */
  uint32_t flags;       /* SKW_KHOP_*                                                  */
  uint64_t seed;
  uint64_t instance_base; /* global id of seed vertex 0 of this call                    */
  uint64_t instance_stride; /* global id of seed i = instance_base + i * instance_stride; 0 = 1 */
} skw_khop_params;

/* Cells per seed in `data` (1 + f1 + f1*f2 ...) and in `sample_lengths` (1 + f1 + ... without
 * the last hop), as Jobs_result<NS>::init computes them (include/sampler_result.cuh:226-260). */
int skw_khop_layout(const skw_khop_params* prm, uint32_t* cells_per_seed,
                    uint32_t* lengths_per_seed);

/* Sample the k-hop neighbourhood tree of n seed vertices.  Replaces OfflineSample
 * (src/offline_sample.cu:443-513) and OnlineGBSampleNew (src/online_sample_new.cu:459-547).
 * data[s * cells + offset(h) + idx]: the child number j of the vertex at (hop h, idx) is at
 * (hop h+1, idx * fanout[h+1] + j) (include/sampler_result.cuh:334-352, 421-426);
 * sample_lengths[s * lens + offset(h) + idx] = children actually sampled from that vertex.
 * Draws are with replacement unless SKW_KHOP_DISTINCT is set.  Cells without a sample hold
 * SKW_INVALID_VERTEX. */
int skw_sample_khop_device(skw_ctx* ctx, const skw_khop_params* prm, const uint32_t* d_seeds,
                           uint64_t n, uint32_t* d_data, uint32_t* d_sample_lengths, float* ms,
                           uint64_t* sampled_edges);
int skw_sample_khop(skw_ctx* ctx, const skw_khop_params* prm, const uint32_t* h_seeds, uint64_t n,
                    uint32_t* h_data, uint32_t* h_sample_lengths, float* ms,
                    uint64_t* sampled_edges);
/* Host buffers, packed result.  No counterpart in the reference, which leaves the tree on the device
 * (include/sampler_result.cuh:334-352).  h_sample_lengths as in skw_sample_khop; h_packed receives,
 * seed after seed, the cells of the seed's row of `data` that hold a sample, in row order (the seed,
 * its hop-1 samples, the hop-2 samples of the first of them, of the second ...): the dense tree
 * without its SKW_INVALID_VERTEX cells, which sample_lengths is enough to rebuild.  *cells = cells
 * the result needs; when capacity_cells is smaller (or h_packed is NULL) the call fills
 * h_sample_lengths and *cells, leaves h_packed unspecified (never written past capacity_cells) and
 * returns SKW_ERR_ARG.  The tree of a power-law graph is sparse (vertices without out-edges have no
 * children), and the host result is bound by the bus: BASELINE config 4 sends 47 MB instead of 79. */
int skw_sample_khop_packed(skw_ctx* ctx, const skw_khop_params* prm, const uint32_t* h_seeds, uint64_t n,
                           uint32_t* h_packed, uint64_t capacity_cells, uint32_t* h_sample_lengths,
                           uint64_t* cells, float* ms, uint64_t* sampled_edges);

/* Measurement aid, no counterpart in the reference: times a dependent chain of random 32-byte loads
 * (the access pattern of a walk step, same load instruction as the record walk) over a scratch
 * buffer of footprint_bytes and reports giga-accesses per second.  This is the ceiling the step
 * kernels run against; it is far below the streaming bandwidth and does not depend on the bytes
 * per access.  Allocates and frees the scratch buffer. */
int skw_probe_random_gather(skw_ctx* ctx, uint64_t footprint_bytes, uint32_t iters,
                            double* gaccesses_per_s);

/* Self-test of the kernels' bounded waits, no counterpart in the reference (whose block-level
 * constructor can spin forever, include/alias_table_new.cuh:637-708): launches a kernel that waits
 * on a barrier nothing signals; the wait must run out after its poll limit (about a millisecond)
 * and the call must return SKW_ERR_DEVICE ("bounded wait ran out") with the context still usable. */
int skw_selftest_bounded_wait(skw_ctx* ctx);

/* ---------------------------------------------------------------- host helpers ----------- */

/* Pinned host memory for the h_* buffers (optional; any host pointer is accepted). */
int skw_host_alloc(size_t bytes, void** out);
void skw_host_free(void* p);

/* Library version, "major.minor". */
const char* skw_version(void);

#ifdef __cplusplus
}
#endif
#endif /* SKYWALKER_B200_H */
