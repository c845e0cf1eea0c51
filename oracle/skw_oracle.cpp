// CPU oracle for the alias-method sampling / random-walk path.  TEST INFRASTRUCTURE ONLY.
//
// Nothing in the shipped library includes, links or calls this file; it is loaded by the tests,
// by the smoke check and by the benchmark's cpu-baseline / reference legs, as the checker and
// as the timed CPU implementation.
//
// Parity status: PARITY UNPINNED at the bit level.  wpybtw/Skywalker is CUDA-only (no CPU code
// for this path), ships no golden vectors or runnable tests (test/alias_table.cu and
// test/tmp.cu target an API that no longer exists), seeds cuRAND XORWOW by thread id and builds
// its tables with unordered float atomics, so its outputs are not reproducible even against
// itself and no output of it can be compared with this file bit for bit.  What is pinned instead:
//   * Philox4x32-10 against the published Random123 known-answer vectors (tests/golden);
//   * the alias construction against the closed-form properties every alias table must have
//     (exact mass conservation in integers, reconstruction of w_i / sum(w) to 1e-6) and against
//     the hand-checkable vectors the reference's smoke programs use (test/tmp.cu:31-42);
//   * the draw / walk / k-hop rules against the reference kernels they restate, cited below;
//   * statistically, against the reference's OWN offline walk kernel, offline 2-hop sampler and
//     unbiased walk run on the GPU (oracle/ref_cuda builds OfflineWalk / sample_kernel_static,
//     OfflineSample / sample_kernel and UnbiasedWalk from the reference sources): fed with tables of this
//     construction their draws follow the edge weights, the walks have the same length and visit
//     statistics as the walks defined here, and the hop-1 sample counts and sampled vertices of
//     the sampler match the take-all rule defined here (tests/test_reference_kernel.py).
//
// Each function cites the reference code it follows (paths inside the reference tree).
// Everything here is deliberately sequential and naive: it is the definition the GPU kernels
// (which use a closed-form parallel formulation) are compared with, bit for bit.
//
// Build: see oracle/Makefile (g++ -O2 -fopenmp -ffp-contract=off).

#include <algorithm>
#include <cmath>
#include <cstdint>
#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <vector>
#ifdef _OPENMP
#include <omp.h>
#include <parallel/algorithm>
#endif

typedef uint32_t u32;
typedef uint64_t u64;

// ------------------------------------------------------------------ Philox4x32-10 ----------
// Salmon et al., "Parallel random numbers: as easy as 1, 2, 3" (SC'11).  The reference draws
// from cuRAND XORWOW seeded by thread id (src/offline_walk.cu:79,103-104); a counter-based
// generator keyed by (seed, walker, step) replaces it so that a walk is a function of its
// inputs only.
static inline void philox_round(u32 c[4], const u32 k[2]) {
  const u64 p0 = (u64)0xD2511F53u * c[0];
  const u64 p1 = (u64)0xCD9E8D57u * c[2];
  const u32 n0 = (u32)(p1 >> 32) ^ c[1] ^ k[0];
  const u32 n1 = (u32)p1;
  const u32 n2 = (u32)(p0 >> 32) ^ c[3] ^ k[1];
  const u32 n3 = (u32)p0;
  c[0] = n0; c[1] = n1; c[2] = n2; c[3] = n3;
}
static inline void philox(u32 c0, u32 c1, u32 c2, u32 c3, u32 k0, u32 k1, u32 out[4]) {
  u32 c[4] = {c0, c1, c2, c3};
  u32 k[2] = {k0, k1};
  for (int r = 0; r < 10; ++r) {
    philox_round(c, k);
    k[0] += 0x9E3779B9u;
    k[1] += 0xBB67AE85u;
  }
  out[0] = c[0]; out[1] = c[1]; out[2] = c[2]; out[3] = c[3];
}

enum : u32 {
  TAG_WALK = 0x57414C4Bu, TAG_KHOP = 0x4B484F50u, TAG_RMAT = 0x524D4154u,
  TAG_WGHT = 0x57474854u, TAG_STRT = 0x53545254u, TAG_PLAW = 0x504C4157u
};
static inline void philox_tagged(u64 seed, u32 tag, u64 unit, u32 c2, u32 c3, u32 out[4]) {
  philox((u32)unit, (u32)(unit >> 32), c2, c3, (u32)seed, (u32)(seed >> 32) ^ tag, out);
}
// 24-bit uniform in [0,1): exact in fp32.
static inline float u01(u32 r) { return (float)(r >> 8) * 5.9604644775390625e-8f; }
static inline u32 mulhi32(u32 a, u32 b) { return (u32)(((u64)a * b) >> 32); }

// ------------------------------------------------------------------ alias construction -----
// Restates loadFromGraph + construct + SaveAliasTable of include/alias_table_new.cuh
// (1077-1132, 1211-1316, 1105-1115): prob_i = w_i * deg / sum(w); slots with prob < 1 ("small")
// are topped up by slots with prob > 1 ("large"); slot i keeps itself with probability prob[i]
// and otherwise yields alias[i].  A vertex whose weights sum to zero is not valid (1081-1090).
//
// The reference pairs smalls and larges speculatively with float atomics, which makes the table
// depend on warp scheduling.  Here the pairing order is fixed (smalls in index order, larges in
// index order, a large that drops below 1 is topped up by the next large -- Vose's sweep) and the
// masses are integers so that every summation order gives the same bits:
//   B      = min(40, 62 - ceil(log2 n))           bits of one bucket, C = 2^B
//   q_i    = trunc(w_i * 2^(B-1-e)), e = floor(log2 max w)   (non-finite / non-positive w -> 0)
//   Q_i    = q_0 + ... + q_(i-1),  W = Q_n
//   K      = (double)(n*C) / (double)W                       (one IEEE division)
//   g(Q)   = n*C if Q == W, else min(n*C, trunc((double)Q * K))
//   M_i    = g(Q_i + q_i) - g(Q_i)
// g is monotone, so M_i >= 0, a zero weight gets exactly zero mass, and the sum telescopes to
// n*C exactly.  prob is the slot's final own mass / C rounded once to fp32.
static inline int ceil_log2_u32(u32 n) {
  int l = 0;
  while (((u64)1 << l) < n) ++l;
  return l;
}
static inline double dbl_pow2(int e) {  // 2^e as a double, e in [-1022, 1023]
  u64 bits = (u64)(e + 1023) << 52;
  double d;
  memcpy(&d, &bits, 8);
  return d;
}
static inline float sane_weight(float w) { return (w > 0.0f && w < INFINITY) ? w : 0.0f; }

// Integer masses of one vertex.  Returns false when the vertex has no usable weight.
static bool vertex_masses(u32 n, const float* w, std::vector<u64>& M, int& B) {
  float wmax = 0.0f;
  for (u32 i = 0; i < n; ++i) wmax = std::max(wmax, sane_weight(w[i]));
  if (n == 0 || wmax == 0.0f) return false;
  B = std::min(40, 62 - ceil_log2_u32(n));
  const u64 C = (u64)1 << B;
  double dmax = (double)wmax;
  u64 bits;
  memcpy(&bits, &dmax, 8);
  const int e = (int)((bits >> 52) & 0x7FF) - 1023;
  const double scale = dbl_pow2(B - 1 - e);
  M.resize(n);
  u64 W = 0;
  for (u32 i = 0; i < n; ++i) {
    M[i] = (u64)((double)sane_weight(w[i]) * scale);  // q_i, exact product, truncated
    W += M[i];
  }
  const u64 nC = (u64)n * C;
  const double K = (double)nC / (double)W;
  u64 Q = 0, gprev = 0;
  for (u32 i = 0; i < n; ++i) {
    Q += M[i];
    u64 g = nC;
    if (Q != W) {
      g = (u64)((double)Q * K);
      if (g > nC) g = nC;
    }
    M[i] = g - gprev;
    gprev = g;
  }
  return true;
}
static inline float mass_to_prob(u64 m, int B) { return (float)((double)m * dbl_pow2(-B)); }

// One vertex: Vose's sweep with FIFO lists.  prob/alias have n entries.  Returns validity.
static bool alias_vertex(u32 n, const float* w, float* prob, u32* alias) {
  std::vector<u64> M;
  int B = 0;
  if (!vertex_masses(n, w, M, B)) {
    for (u32 i = 0; i < n; ++i) { prob[i] = 1.0f; alias[i] = i; }
    return false;
  }
  const u64 C = (u64)1 << B;
  std::vector<u32> small, large;
  for (u32 i = 0; i < n; ++i) (M[i] < C ? small : large).push_back(i);
  size_t si = 0, li = 0;
  u64 R = M[large[0]];  // what the current donor still owns (sum M == n*C => a large exists)
  for (;;) {
    if (R >= C && si < small.size()) {
      const u32 s = small[si++];            // donor tops up the next small
      prob[s] = mass_to_prob(M[s], B);
      alias[s] = large[li];
      R -= C - M[s];
    } else if (R < C) {
      const u32 l = large[li];              // donor fell below one bucket: it becomes a
      prob[l] = mass_to_prob(R, B);         // bucket itself, topped up by the next large
      alias[l] = large[li + 1];
      R = M[large[li + 1]] - (C - R);
      ++li;
    } else {                                // no small left and the donor owns a full bucket
      const u32 l = large[li];
      prob[l] = 1.0f;
      alias[l] = l;
      if (++li == large.size()) break;
      R = M[large[li]];
    }
  }
  return true;
}

extern "C" {

void orc_philox4x32_10(const u32 ctr[4], const u32 key[2], u32 out[4]) {
  philox(ctr[0], ctr[1], ctr[2], ctr[3], key[0], key[1], out);
}

int orc_num_threads(void) {
#ifdef _OPENMP
  return omp_get_max_threads();
#else
  return 1;
#endif
}
void orc_free(void* p) { free(p); }

int orc_alias_build_vertex(u32 n, const float* w, float* prob, u32* alias) {
  return alias_vertex(n, w, prob, alias) ? 1 : 0;
}

// Integer masses of one vertex (for the mass-conservation test).  Returns B or -1.
int orc_alias_vertex_masses(u32 n, const float* w, u64* M_out) {
  std::vector<u64> M;
  int B = 0;
  if (!vertex_masses(n, w, M, B)) return -1;
  memcpy(M_out, M.data(), sizeof(u64) * n);
  return B;
}

// All vertices of [v_begin, v_end): ConstructTable (src/createTable.cu:119-179).  prob/alias are
// indexed like the CSR (slot xadj[v] + i), valid per vertex.
void orc_alias_build(u32 v_begin, u32 v_end, const u32* xadj, const float* adjwgt, float* prob,
                     u32* alias, uint8_t* valid, int threads) {
#pragma omp parallel for schedule(dynamic, 256) num_threads(threads > 0 ? threads : orc_num_threads())
  for (long long v = v_begin; v < (long long)v_end; ++v) {
    const u32 off = xadj[v], n = xadj[v + 1] - off;
    valid[v] = alias_vertex(n, adjwgt + off, prob + off, alias + off) ? 1 : 0;
  }
}

// Largest relative error of the probabilities a table encodes:
// P(j) = (prob[j] + sum_{i != j, alias[i] == j} (1 - prob[i])) / deg  against  w_j / sum(w).
double orc_alias_reconstruct_maxrel(u32 V, const u32* xadj, const float* adjwgt, const float* prob,
                                    const u32* alias, const uint8_t* valid) {
  double worst = 0.0;
#pragma omp parallel
  {
    std::vector<double> acc;
    double mine = 0.0;
#pragma omp for schedule(dynamic, 256)
    for (long long v = 0; v < (long long)V; ++v) {
      if (!valid[v]) continue;
      const u32 off = xadj[v], n = xadj[v + 1] - off;
      acc.assign(n, 0.0);
      double W = 0.0;
      for (u32 i = 0; i < n; ++i) {
        W += (double)sane_weight(adjwgt[off + i]);
        acc[i] += (double)prob[off + i];
        const u32 a = alias[off + i];
        if (a >= n) { mine = 1e30; continue; }
        if (a != i) acc[a] += 1.0 - (double)prob[off + i];
      }
      for (u32 i = 0; i < n; ++i) {
        const double want = (double)sane_weight(adjwgt[off + i]) / W;
        const double got = acc[i] / (double)n;
        const double err = want > 0.0 ? std::fabs(got - want) / want : std::fabs(got);
        if (err > mine) mine = err;
      }
    }
#pragma omp critical
    if (mine > worst) worst = mine;
  }
  return worst;
}

// ------------------------------------------------------------------ draws ------------------
// The alias draw of sample_kernel_static (src/offline_walk.cu:100-112): a column, a uniform,
// keep the column if the uniform is below its prob, else take its alias.  The column comes from
// a 32-bit multiply-high instead of floor(curand_uniform * deg), which can return deg because
// curand_uniform is in (0,1].
static inline u32 alias_draw(const float* prob, const u32* alias, u32 deg, u32 r_col, u32 r_acc) {
  const u32 col = mulhi32(r_col, deg);
  return u01(r_acc) < prob[col] ? col : alias[col];
}

// bool CheckConnect(src, dst): binary search of dst in the sorted adjacency of src
// (include/gpu_graph.cuh:204-238).
static inline bool connected(const u32* xadj, const u32* adjncy, u32 src, u32 dst) {
  const u32* b = adjncy + xadj[src];
  const u32* e = adjncy + xadj[src + 1];
  return std::binary_search(b, e, dst);
}

enum { APP_DEEPWALK = 0, APP_PPR = 1, APP_NODE2VEC = 2 };
enum { N2V_MAX_TRIALS = 64 };

// One walker.  Follows sample_kernel_static (src/offline_walk.cu:75-124): degree 0 ends the walk
// with length = step; degree 1 takes the only neighbour; otherwise one alias draw.  PPR adds the
// test of src/online_walk.cu:109-125 / src/unbiased_walk.cu:82 before every step.  node2vec
// follows Node2vecKernelStaticBuffer (src/unbiased_walk.cu:14-61) with the weights of
// src/api/bias_node2vec.cu:14-24: propose from the static table, accept with probability
// f / max(1/p, 1, 1/q), f = 1/p back to the previous vertex, 1 to a neighbour of it, 1/q else.
// online != 0 rebuilds the table of the current vertex from its weights at every step, as
// OnlineWalkKernel does (src/online_walk.cu:10-40), instead of reading the stored one.
// unbiased != 0: the neighbour is drawn uniformly (column only, no table), as UnbiasedWalkKernelStatic
// does (src/unbiased_walk.cu:102-124); node2vec then is exactly Node2vecKernelStaticBuffer.
static void walk_one(const u32* xadj, const u32* adjncy, const float* adjwgt, const float* prob,
                     const u32* alias, const uint8_t* valid, int online, int unbiased, int app, u32 hop_num,
                     float tp, float inv_p, float inv_q, u64 seed, u64 gw, u32 start, u32* row,
                     u32* length, std::vector<float>& tprob, std::vector<u32>& talias) {
  const float fmax = std::max(1.0f, std::max(inv_p, inv_q));
  u32 cur = start, prev = 0xFFFFFFFFu;
  row[0] = start;
  u32 step = 0;
  for (; step + 1 < hop_num; ++step) {
    u32 r[4];
    philox_tagged(seed, TAG_WALK, gw, step, 0, r);
    if (app == APP_PPR && u01(r[2]) < tp) break;
    const u32 off = xadj[cur], deg = xadj[cur + 1] - off;
    if (deg == 0) break;
    const float* vp = nullptr;
    const u32* va = nullptr;
    if (unbiased) {
    } else if (online) {
      tprob.resize(deg);
      talias.resize(deg);
      if (!alias_vertex(deg, adjwgt + off, tprob.data(), talias.data())) break;
      vp = tprob.data();
      va = talias.data();
    } else {
      if (!valid[cur]) break;
      vp = prob + off;
      va = alias + off;
    }
    u32 next;
    if (app == APP_NODE2VEC && prev != 0xFFFFFFFFu) {
      u32 trial = 0;
      for (;;) {
        const u32 cand = unbiased ? mulhi32(r[0], deg) : (deg == 1 ? 0 : alias_draw(vp, va, deg, r[0], r[1]));
        next = adjncy[off + cand];
        const float f = next == prev ? inv_p : (connected(xadj, adjncy, prev, next) ? 1.0f : inv_q);
        if (u01(r[3]) * fmax < f) break;
        if (++trial == N2V_MAX_TRIALS) break;  // keep the last proposal
        philox_tagged(seed, TAG_WALK, gw, step, trial, r);
      }
    } else {
      const u32 cand = unbiased ? mulhi32(r[0], deg) : (deg == 1 ? 0 : alias_draw(vp, va, deg, r[0], r[1]));
      next = adjncy[off + cand];
    }
    row[step + 1] = next;
    prev = cur;
    cur = next;
  }
  *length = step;
}

// n walkers; paths[w * hop_num + s], lengths[w] (include/sampler_result.cuh:607-612).
// Cells after paths[w*hop_num + lengths[w]] are left untouched.
void orc_walk(const u32* xadj, const u32* adjncy, const float* adjwgt, const float* prob,
              const u32* alias, const uint8_t* valid, int online, int unbiased, int app, u32 hop_num, float tp,
              float p, float q, u64 seed, u64 walker_base, u64 walker_stride, const u32* starts, u64 n,
              u32* paths, u32* lengths, int threads) {
  const float inv_p = 1.0f / p, inv_q = 1.0f / q;
#pragma omp parallel num_threads(threads > 0 ? threads : orc_num_threads())
  {
    std::vector<float> tprob;
    std::vector<u32> talias;
#pragma omp for schedule(dynamic, 64)
    for (long long w = 0; w < (long long)n; ++w)
      walk_one(xadj, adjncy, adjwgt, prob, alias, valid, online, unbiased, app, hop_num, tp, inv_p, inv_q,
               seed, walker_base + (u64)w * walker_stride, starts[w], paths + (u64)w * hop_num, lengths + w, tprob,
               talias);
  }
}

// ------------------------------------------------------------------ k-hop ------------------
// Result tree of Jobs_result<NS> (include/sampler_result.cuh:226-260, 334-352, 421-426) filled
// the way the offline sampler does (src/offline_sample.cu:72-141): for every vertex of hop h draw
// fanout[h+1] neighbours with replacement from its table; with take_all, a vertex whose degree
// is <= the fan-out contributes each neighbour once instead (120-128).  Cells without a sample
// hold 0xFFFFFFFF.  fanout[0..nhops-1] are the reference's hops[1..].
//
// flags & 4 (distinct): the rule of the reference's ONLINE sampler, roll_atomic / roll_once
// (src/online_sample_new.cu:73-111, 3-37): a vertex whose degree is <= the fan-out contributes every
// neighbour once; otherwise columns are drawn from the table and a draw counts only if its column was
// not drawn before, until fan-out distinct columns are found or the trials run out.  The reference
// lets the 32 lanes of a warp draw at once for at most 11 rounds, in whatever order the atomics land;
// here the 352 trials are numbered (trial t = lane + 32 * round) and taken in that order, each with
// its own Philox words keyed by (seed id, parent index, trial, hop), so the result is reproducible.
// The sample length is the number of distinct columns found.
enum { KHOP_DISTINCT_TRIALS = 352 };  // 32 lanes x 11 rounds (src/online_sample_new.cu:86-96)

void orc_khop(const u32* xadj, const u32* adjncy, const float* adjwgt, const float* prob,
              const u32* alias, const uint8_t* valid, int online, u32 nhops, const u32* fanout,
              u32 flags, u64 seed, u64 instance_base, u64 instance_stride, const u32* seeds, u64 n,
              u32* data, u32* sample_lengths, int threads) {
  u32 width[8], offs[8];
  u32 cells = 0, w = 1;
  for (u32 h = 0; h <= nhops; ++h) {
    if (h) w *= fanout[h - 1];
    width[h] = w;
    offs[h] = cells;
    cells += w;
  }
  const u32 lens = offs[nhops];
#pragma omp parallel num_threads(threads > 0 ? threads : orc_num_threads())
  {
    std::vector<float> tprob;
    std::vector<u32> talias;
#pragma omp for schedule(dynamic, 16)
    for (long long s = 0; s < (long long)n; ++s) {
      u32* row = data + (u64)s * cells;
      u32* len = sample_lengths + (u64)s * lens;
      const u64 gi = instance_base + (u64)s * instance_stride;
      row[0] = seeds[s];
      for (u32 h = 0; h < nhops; ++h) {
        const u32 f = fanout[h];
        for (u32 idx = 0; idx < width[h]; ++idx) {
          const u32 v = row[offs[h] + idx];
          u32* child = row + offs[h + 1] + (u64)idx * f;
          u32 got = 0;
          const float* vp = nullptr;
          const u32* va = nullptr;
          u32 off = 0, deg = 0;
          bool ok = v != 0xFFFFFFFFu;
          if (ok) {
            off = xadj[v];
            deg = xadj[v + 1] - off;
            ok = deg > 0;
          }
          if (ok) {
            // distinct draws are a rule of the biased sampler; with the unbiased flag it is ignored
            const bool distinct = (flags & 4u) && !(flags & 2u);
            if (((flags & 1u) || distinct) && f >= deg) {
              for (u32 j = 0; j < deg; ++j) child[j] = adjncy[off + j];
              got = deg;
            } else if (flags & 2u) {  // unbiased: uniform column, no table (src/unbiased_sample.cu:28-36)
              for (u32 j = 0; j < f; ++j) {
                u32 r[4];
                philox_tagged(seed, TAG_KHOP, gi, idx * f + j, h + 1, r);
                child[j] = adjncy[off + mulhi32(r[0], deg)];
              }
              got = f;
            } else {
              if (online) {
                tprob.resize(deg);
                talias.resize(deg);
                ok = alias_vertex(deg, adjwgt + off, tprob.data(), talias.data());
                vp = tprob.data();
                va = talias.data();
              } else {
                ok = valid[v] != 0;
                vp = prob + off;
                va = alias + off;
              }
              if (ok && distinct) {
                std::vector<u32> seen;
                for (u32 t = 0; t < KHOP_DISTINCT_TRIALS && got < f; ++t) {
                  u32 r[4];
                  philox_tagged(seed, TAG_KHOP, gi, idx, (t << 8) | 0x80u | (h + 1), r);
                  const u32 c = alias_draw(vp, va, deg, r[0], r[1]);
                  if (std::find(seen.begin(), seen.end(), c) != seen.end()) continue;
                  seen.push_back(c);
                  child[got++] = adjncy[off + c];
                }
              } else if (ok) {
                for (u32 j = 0; j < f; ++j) {
                  u32 r[4];
                  philox_tagged(seed, TAG_KHOP, gi, idx * f + j, h + 1, r);
                  child[j] = adjncy[off + alias_draw(vp, va, deg, r[0], r[1])];
                }
                got = f;
              }
            }
          }
          for (u32 j = got; j < f; ++j) child[j] = 0xFFFFFFFFu;
          len[offs[h] + idx] = got;
        }
      }
    }
  }
}

// ------------------------------------------------------------------ synthetic inputs -------
static inline u32 scramble(u32 v, u32 scale) {
  const u32 mask = scale >= 32 ? 0xFFFFFFFFu : ((1u << scale) - 1u);
  const u32 sh = scale / 2 ? scale / 2 : 1;
  v = (v * 0x9E3779B1u) & mask;
  v ^= v >> sh;
  v = (v * 0x85EBCA6Bu) & mask;
  v ^= v >> sh;
  return v;
}

static void keys_to_csr(std::vector<u64>& keys, u32 V, u32** xadj_out, u32** adjncy_out,
                        u64* E_out) {
#ifdef _OPENMP
  __gnu_parallel::sort(keys.begin(), keys.end());
#else
  std::sort(keys.begin(), keys.end());
#endif
  keys.erase(std::unique(keys.begin(), keys.end()), keys.end());
  if (!keys.empty() && keys.back() == ~(u64)0) keys.pop_back();
  const u64 E = keys.size();
  u32* xadj = (u32*)calloc((size_t)V + 1, sizeof(u32));
  u32* adj = (u32*)malloc(sizeof(u32) * (E ? E : 1));
  for (u64 i = 0; i < E; ++i) {
    xadj[(keys[i] >> 32) + 1]++;
    adj[i] = (u32)keys[i];
  }
  for (u32 v = 0; v < V; ++v) xadj[v + 1] += xadj[v];
  *xadj_out = xadj;
  *adjncy_out = adj;
  *E_out = E;
}

// Seeded R-MAT (Chakrabarti et al.): raw_edges draws of `scale` quadrant choices each, one 32-bit
// Philox word per level compared with integer thresholds; ids scrambled; self loops and
// duplicates removed; adjacency sorted.
int orc_gen_rmat(u32 scale, u32 num_vertices, u64 raw_edges, double a, double b, double c,
                 int symmetric, u64 seed, u32* V_out, u64* E_out, u32** xadj_out, u32** adjncy_out) {
  if (scale < 1 || scale > 31) return -1;
  const u32 ta = (u32)std::min(4294967295.0, a * 4294967296.0);
  const u32 tab = (u32)std::min(4294967295.0, (a + b) * 4294967296.0);
  const u32 tabc = (u32)std::min(4294967295.0, (a + b + c) * 4294967296.0);
  const u32 fold = (num_vertices && num_vertices < (1u << scale)) ? num_vertices : 0;
  const u64 per = symmetric ? 2 : 1;
  std::vector<u64> keys(raw_edges * per);
#pragma omp parallel for schedule(static)
  for (long long ee = 0; ee < (long long)raw_edges; ++ee) {
    const u64 e = (u64)ee;
    u32 src = 0, dst = 0, r[4];
    for (u32 l = 0; l < scale; ++l) {
      if ((l & 3) == 0) philox_tagged(seed, TAG_RMAT, e, l >> 2, 0, r);
      const u32 x = r[l & 3];
      const u32 sb = x >= tab ? 1u : 0u;
      const u32 db = (x >= ta && x < tab) || x >= tabc ? 1u : 0u;
      src = (src << 1) | sb;
      dst = (dst << 1) | db;
    }
    src = scramble(src, scale);
    dst = scramble(dst, scale);
    if (fold) {
      src %= fold;
      dst %= fold;
    }
    const bool loop = src == dst;  // self loops become a sentinel that sorts last
    keys[e * per] = loop ? ~(u64)0 : (((u64)src << 32) | dst);
    if (symmetric) keys[e * per + 1] = loop ? ~(u64)0 : (((u64)dst << 32) | src);
  }
  *V_out = fold ? fold : 1u << scale;
  keys_to_csr(keys, *V_out, xadj_out, adjncy_out, E_out);
  return 0;
}

// Target degrees of the power-law generator: min(cap, floor(dmin * u^(-1/(exponent-1)))),
// u = (24-bit Philox draw + 1) / 2^24; cum[v+1] - cum[v] = target degree of v.
void orc_powerlaw_targets(u32 V, double exponent, double dmin, u32 cap, u64 seed, u64* cum) {
  cum[0] = 0;
  const double ex = -1.0 / (exponent - 1.0);
  for (u32 v = 0; v < V; ++v) {
    u32 r[4];
    philox_tagged(seed, TAG_PLAW, v, 0, 1, r);
    const double u = ((double)(r[0] >> 8) + 1.0) * 5.9604644775390625e-8;
    double d = std::floor(dmin * std::pow(u, ex));
    if (!(d < (double)cap)) d = (double)cap;
    if (d < 1.0) d = 1.0;
    cum[v + 1] = cum[v] + (u64)d;
  }
}

static inline u64 mulhi64(u64 a, u64 b) { return (u64)(((unsigned __int128)a * b) >> 64); }

int orc_gen_powerlaw(u32 V, u64 raw_edges, double exponent, double dmin, u32 cap, u64 seed,
                     u64* E_out, u32** xadj_out, u32** adjncy_out) {
  std::vector<u64> cum((size_t)V + 1);
  orc_powerlaw_targets(V, exponent, dmin, cap, seed, cum.data());
  const u64 S = cum[V];
  std::vector<u64> keys(raw_edges * 2);
#pragma omp parallel for schedule(static)
  for (long long ee = 0; ee < (long long)raw_edges; ++ee) {
    const u64 e = (u64)ee;
    u32 r[4];
    philox_tagged(seed, TAG_PLAW, e, 0, 0, r);
    const u64 x = mulhi64(((u64)r[0] << 32) | r[1], S);
    const u64 y = mulhi64(((u64)r[2] << 32) | r[3], S);
    const u32 a = (u32)(std::upper_bound(cum.begin(), cum.end(), x) - cum.begin() - 1);
    const u32 b = (u32)(std::upper_bound(cum.begin(), cum.end(), y) - cum.begin() - 1);
    keys[2 * e] = a == b ? ~(u64)0 : (((u64)a << 32) | b);
    keys[2 * e + 1] = a == b ? ~(u64)0 : (((u64)b << 32) | a);
  }
  keys_to_csr(keys, V, xadj_out, adjncy_out, E_out);
  return 0;
}

// Edge weights: 1 + 9 * k / 2^24 rounded down to a multiple of 2^-20 (k = 24-bit draw of edge e).
void orc_gen_weights(u64 E, u64 seed, float* w) {
#pragma omp parallel for schedule(static)
  for (long long e = 0; e < (long long)E; ++e) {
    u32 r[4];
    philox_tagged(seed, TAG_WGHT, (u64)e, 0, 0, r);
    const u32 val = (1u << 20) + (((r[0] >> 8) * 9u) >> 4);
    w[e] = (float)val * 9.5367431640625e-7f;
  }
}

void orc_gen_starts(u64 n, u64 id_base, u32 V, u64 seed, u32* starts) {
  for (u64 i = 0; i < n; ++i) {
    u32 r[4];
    philox_tagged(seed, TAG_STRT, id_base + i, 0, 0, r);
    starts[i] = mulhi32(r[0], V);
  }
}

}  // extern "C"
