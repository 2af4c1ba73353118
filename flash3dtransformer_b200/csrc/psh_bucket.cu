// Batched perfect-spatial-hash bucketing and scatter for sm_100a.
//
// Replaces the reference's three kernels
//   batch_psh_bucketing_balancing_ker     src/psh/batch_psh_bucket.cuh:42-257
//   batch_psh_distribute_recycle_ker      src/psh/batch_psh_bucket.cuh:259-382
//   batch_psh_cumsum_scatter_postpad_ker  src/psh/batch_psh_bucket.cuh:493-614
// and their host driver batch_psh_scatter_pad_hash (src/psh/batch_psh_bucket_dispatcher.cu:221-326).
//
// The reference decides in-bucket offsets by atomicInc arrival order and rebalances with racy reads, so its
// output differs from run to run.  Here every offset is a *stable rank by input index*, which is one of the
// outcomes the reference can produce for points that do not overflow, and the rebalance is defined as three
// deterministic rounds (scene-local, input order = index order inside the scene):
//
//   round A  bucket b = first_hash(vox).  rank_A = number of earlier points of the scene with the same b.
//            A point keeps (b, rank_A) if b is the recycle bucket 0 or rank_A < bucket_size.
//            kept[b] = count[b] for b == 0, min(count[b], bucket_size) otherwise.
//   round B  every other point makes one attempt, as in the reference (one attempt per point because the
//            segment commit test at batch_psh_bucket.cuh:218 only fires on the last probe): it walks the 128
//            probes in table order and takes the first perturbed-hash bucket t that is neither its own bucket
//            nor bucket 0 and has kept[t] < bucket_size.  Attempts on t are ranked by input index; the first
//            bucket_size - kept[t] are accepted at offset kept[t] + rank_B.  The rest, and points with no
//            admissible probe, go to the recycle bucket at offset count[0] + (rejected of lower t) + (rank_B -
//            free[t]); points without a probe are ordered last.
//   round C  recycle-bucket points at offset >= bucket_size are redistributed as in the recycle kernel: one
//            random probe, perturbed hash, a random non-zero bucket if that hashes to 0, no capacity check.
//            Arrivals on bucket c are ranked by input index and appended after round B's content of c.
//
// Each round is "tile histogram -> per-scene scan over tiles -> tile rank", so a point's rank needs no atomics
// on global memory and no inter-CTA waiting: seven launches (key + histogram, scan, round A ranks + probe walk, scan,
// round B resolution, scan, round C ranks + scatter) over tiles of 2048 points, so that even one scan of 120,000
// points spreads over 59 CTAs and a batch fills every SM.  The first-hash key of a point is computed once (kernel 1)
// and kept as 16 bits in scratch; the rank kernels read keys, not coordinates.  The scan kernel turns a round's table
// of per-tile counts into per-tile exclusive prefixes in place, one warp per (scene, bucket) column, and writes the
// scene totals.  Warps own contiguous index ranges; equal keys inside a warp are merged with match_any
// (warp-aggregated counting), per-warp counters live in shared memory, and coordinates are staged into shared memory
// with 128-bit loads where they are needed (kernel 1, the probe walk of overflowing points, the scatter).
#include "f3d_common.cuh"
#include <map>
#include <mutex>
#include "psh_device.cuh"
#include "../../include/f3d_b200.h"

namespace f3d {

uint64_t seed();
uint32_t scene_base();

constexpr int kPshThreads = 256;
constexpr int kPshWarps = kPshThreads / 32;
constexpr uint32_t kGroup = 256;            // points one warp stages at a time
constexpr uint32_t kStageHalves = kGroup * 3 + 16;   // staged halves + room for the 16-byte alignment skew
constexpr uint32_t kDefaultTile = 2048;     // points per tile (one CTA)
constexpr uint32_t kMinTile = 256;          // a warp's slice of a tile is at least 32 points
constexpr uint32_t kMaxTile = 16384;
constexpr size_t kFewTiles = 148;           // batches with fewer tiles than this take smaller tiles

// Jump constants of the probe streams, s_n = A^n s_0 + C_n (mod 2^32) for the linear congruential step
// s <- 1664525 s + 1013904223: entry n - 1 holds (A^n, C_n), n = 1 .. 128, evaluated at compile time.
struct LcgJumps { uint32_t a[kNumProbes], c[kNumProbes]; };
constexpr LcgJumps make_lcg_jumps() {
  LcgJumps j{};
  uint32_t pa = 1u, pc = 0u;
  for (uint32_t n = 0; n < kNumProbes; ++n) {
    pa *= 1664525u;
    pc = pc * 1664525u + 1013904223u;
    j.a[n] = pa; j.c[n] = pc;
  }
  return j;
}
__constant__ LcgJumps g_lcg_jumps = make_lcg_jumps();

struct PshArgs {
  const __half *coord; uint16_t *bucket_id; uint32_t *bucket_counter; uint32_t *bucket_offset;
  const uint32_t *batch_sep; uint32_t *cumsum_counter; __half *scatter_coord;
  const __half *bbox_min; const __half *bbox_max; const int16_t *probe;
  uint32_t total_N, batch, nb, nbp, divisor, cap, num_vox, hash_type, pad_to;
  uint32_t tile, tiles_max;
  uint16_t pad_bits; uint16_t coord_aligned; uint16_t out_aligned;
  RngKey key;
  uint32_t scene_base;     // added to the scene index in the random-number counter (global scene id of a shard)
  // scratch
  uint32_t *tabA, *tabB, *tabC;    // [batch][nbp][tiles_max] tile tables of rounds A, B, C: raw counts, then (after the
                                   // round's scan) the exclusive prefix over the scene's earlier tiles.  A (scene,
                                   // bucket) column is contiguous, so the scan reads and writes whole lines; the
                                   // tile kernels touch one word per column
  uint32_t *count0, *kept, *cntB;  // [batch][nbp] first-hash totals, kept counts, counts after round B
  uint32_t *attB, *movC;           // [batch][nbp] scene totals of the round B attempts and the round C movers
  uint32_t *tile_pending, *tile_movers;                     // [batch*tiles_max]
  uint16_t *keys;                  // [total_N] first-hash key of every point
};

// ---------------------------------------------------------------------------------------------------------
// shared-memory plan of the tile kernels
struct TileSmem {
  uint16_t *stage;     // [kPshWarps][kStageHalves]
  uint16_t *whist;     // [kPshWarps][nbp]   per-warp counts, then per-warp running ranks (tile-relative)
  uint32_t *tbase;     // [nbp]              rank of the tile's first element of each key
  uint32_t *aux;       // [nbp]              block histogram of the next round / cached per-scene table
  uint32_t *aux2;      // [nbp]              second cached per-scene table
  uint32_t *aux3;      // [nbp]              third cached per-scene table
  uint32_t *aux4;      // [nbp]              this tile's histogram of the next round (flushed with plain stores)
  uint16_t *keys;      // [tile]             key cache between the counting and the ranking sweep
};

__host__ __device__ inline size_t tile_smem_bytes(uint32_t nbp, uint32_t tile) {
  size_t b = 0;
  b += (size_t)kPshWarps * kStageHalves * 2;
  b += ((size_t)kPshWarps * nbp * 2 + 15) / 16 * 16;
  b += (size_t)nbp * 4 * 5;
  b += (size_t)tile * 2;
  return b + 64;
}

__device__ __forceinline__ TileSmem carve(unsigned char *base, uint32_t nbp, uint32_t tile) {
  TileSmem s;
  s.stage = reinterpret_cast<uint16_t *>(base);
  base += (size_t)kPshWarps * kStageHalves * 2;          // multiple of 16
  s.whist = reinterpret_cast<uint16_t *>(base);
  base += ((size_t)kPshWarps * nbp * 2 + 15) / 16 * 16;
  s.tbase = reinterpret_cast<uint32_t *>(base);
  base += (size_t)nbp * 4;
  s.aux = reinterpret_cast<uint32_t *>(base);
  base += (size_t)nbp * 4;
  s.aux2 = reinterpret_cast<uint32_t *>(base);
  base += (size_t)nbp * 4;
  s.aux3 = reinterpret_cast<uint32_t *>(base);
  base += (size_t)nbp * 4;
  s.aux4 = reinterpret_cast<uint32_t *>(base);
  base += (size_t)nbp * 4;
  s.keys = reinterpret_cast<uint16_t *>(base);
  return s;
}

// Stage points [g, g+cnt) of the flat [N,3] fp16 array into the warp's shared buffer with 128-bit loads.
// Returns the offset (in halves) of point g inside the buffer.
__device__ __forceinline__ uint32_t warp_stage(const PshArgs &a, uint32_t g, uint32_t cnt, uint16_t *dst, int lane) {
  const uint16_t *src = reinterpret_cast<const uint16_t *>(a.coord);
  const uint64_t total_h = (uint64_t)a.total_N * 3ull;
  uint64_t h0 = (uint64_t)g * 3ull, h1 = h0 + (uint64_t)cnt * 3ull;
  __syncwarp();
  if (a.coord_aligned) {
    uint64_t a0 = h0 & ~7ull;                       // 8 halves = 16 bytes
    uint32_t nvec = (uint32_t)((h1 - a0 + 7ull) / 8ull);
    for (uint32_t v = lane; v < nvec; v += 32) {
      uint64_t off = a0 + (uint64_t)v * 8ull;
      if (off + 8ull <= total_h) {
        uint4 w = __ldg(reinterpret_cast<const uint4 *>(src + off));
        *reinterpret_cast<uint4 *>(dst + v * 8u) = w;
      } else {
        for (uint32_t e = 0; e < 8 && off + e < total_h; ++e) dst[v * 8u + e] = src[off + e];
      }
    }
    __syncwarp();
    return (uint32_t)(h0 - a0);
  }
  for (uint32_t e = lane; e < cnt * 3u; e += 32) dst[e] = src[h0 + e];
  __syncwarp();
  return 0u;
}

__device__ __forceinline__ void load_vox(const uint16_t *st, uint32_t skew, uint32_t k, const AxisScale (&ax)[3],
                                         uint32_t (&vox)[3]) {
#pragma unroll
  for (int d = 0; d < 3; ++d) vox[d] = vox_axis(__half2float(__ushort_as_half(st[skew + 3u * k + d])), ax[d]);
}

__device__ __forceinline__ void load_axes(const PshArgs &a, AxisScale (&ax)[3]) {
#pragma unroll
  for (int d = 0; d < 3; ++d) ax[d] = make_axis_scale(__half2float(a.bbox_min[d]), __half2float(a.bbox_max[d]), a.num_vox);
}

struct TileInfo { uint32_t scene, tile, start, n, t0, cnt, row; bool live; };

// word of a tile table for (scene, bucket column, tile)
__device__ __forceinline__ size_t tab_at(const PshArgs &a, uint32_t scene, uint32_t col, uint32_t tile) {
  return ((size_t)scene * a.nbp + col) * a.tiles_max + tile;
}

__device__ __forceinline__ TileInfo tile_info(const PshArgs &a) {
  TileInfo t;
  t.scene = blockIdx.y; t.tile = blockIdx.x;
  t.start = t.scene ? a.batch_sep[t.scene - 1] : 0u;
  uint32_t end = a.batch_sep[t.scene];
  if (end > a.total_N) end = a.total_N;
  t.n = end > t.start ? end - t.start : 0u;
  t.t0 = t.tile * a.tile;
  t.live = t.t0 < t.n;
  t.cnt = t.live ? min(a.tile, t.n - t.t0) : 0u;
  t.row = t.scene * a.tiles_max + t.tile;
  return t;
}

// warp-aggregated counting of one key per lane (all 32 lanes call)
__device__ __forceinline__ void warp_count(uint16_t *wh, uint32_t key, bool valid, int lane) {
  uint32_t peers = __match_any_sync(0xFFFFFFFFu, valid ? key : 0xFFFFFFFFu);
  if (valid && (__ffs(peers) - 1) == lane) wh[key] = (uint16_t)(wh[key] + __popc(peers));
  __syncwarp();
}

// stable rank of one key per lane; wh holds the warp's running tile-relative rank of every key
__device__ __forceinline__ uint32_t warp_rank(uint16_t *wh, const uint32_t *tbase, uint32_t key, bool valid, int lane) {
  uint32_t peers = __match_any_sync(0xFFFFFFFFu, valid ? key : 0xFFFFFFFFu);
  uint32_t base = valid ? wh[key] : 0u;
  __syncwarp();
  if (valid && (__ffs(peers) - 1) == lane) wh[key] = (uint16_t)(base + __popc(peers));
  __syncwarp();
  uint32_t lower = __popc(peers & ((1u << lane) - 1u));
  return valid ? tbase[key] + base + lower : 0u;
}

__device__ __forceinline__ void zero_whist(const TileSmem &s, uint32_t nbp) {
  for (uint32_t i = threadIdx.x; i < kPshWarps * nbp; i += kPshThreads) s.whist[i] = 0;
}

// per-warp counts -> per-warp exclusive prefix (tile-relative)
__device__ __forceinline__ void warp_prefix(const TileSmem &s, uint32_t nbp) {
  for (uint32_t b = threadIdx.x; b < nbp; b += kPshThreads) {
    uint32_t run = 0;
#pragma unroll
    for (int w = 0; w < kPshWarps; ++w) {
      uint32_t c = s.whist[w * nbp + b];
      s.whist[w * nbp + b] = (uint16_t)run;
      run += c;
    }
  }
}

// ---------------------------------------------------------------------------------------------------------
// K1: first-hash key of every point (kept in scratch) and the key histogram of every tile
__global__ void __launch_bounds__(kPshThreads) psh_hist_kernel(PshArgs a) {
  extern __shared__ __align__(16) unsigned char smem_raw[];
  TileSmem s = carve(smem_raw, a.nbp, 0);
  TileInfo t = tile_info(a);
  if (!t.live) return;
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  for (uint32_t b = threadIdx.x; b < a.nbp; b += kPshThreads) s.aux[b] = 0;
  __syncthreads();
  AxisScale ax[3];
  load_axes(a, ax);
  const HashPlan hp = make_hash_plan(a.hash_type, a.divisor, a.nb);
  const uint32_t wt = a.tile / kPshWarps;
  const uint32_t w0 = warp * wt, w1 = min(w0 + wt, t.cnt);
  uint16_t *st = s.stage + warp * kStageHalves;
  uint16_t *keys = a.keys + t.start + t.t0;
  for (uint32_t g = w0; g < w1; g += kGroup) {
    uint32_t gc = min(kGroup, w1 - g);
    uint32_t skew = warp_stage(a, t.start + t.t0 + g, gc, st, lane);
    for (uint32_t it = 0; it < gc; it += 32) {
      uint32_t k = it + lane;
      bool valid = k < gc;
      uint32_t key = 0;
      if (valid) {
        uint32_t vox[3];
        load_vox(st, skew, k, ax, vox);
        key = first_hash(hp, vox[0], vox[1], vox[2]);
        keys[g + k] = (uint16_t)key;
      }
      uint32_t peers = __match_any_sync(0xFFFFFFFFu, valid ? key : 0xFFFFFFFFu);
      if (valid && (__ffs(peers) - 1) == lane) atomicAdd(&s.aux[key], (uint32_t)__popc(peers));
    }
  }
  __syncthreads();
  for (uint32_t b = threadIdx.x; b < a.nbp; b += kPshThreads) a.tabA[tab_at(a, t.scene, b, t.tile)] = s.aux[b];
}

// ---------------------------------------------------------------------------------------------------------
// block-wide exclusive scan of one value per thread (kPshThreads threads); returns exclusive prefix, total in *tot
__device__ __forceinline__ uint32_t block_excl_scan(uint32_t v, uint32_t *wsum /*[kPshWarps+1]*/, uint32_t *tot) {
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  uint32_t inc = v;
#pragma unroll
  for (int d = 1; d < 32; d <<= 1) {
    uint32_t o = __shfl_up_sync(0xFFFFFFFFu, inc, d);
    if (lane >= d) inc += o;
  }
  if (lane == 31) wsum[warp] = inc;
  __syncthreads();
  if (threadIdx.x == 0) {
    uint32_t run = 0;
    for (int w = 0; w < kPshWarps; ++w) { uint32_t c = wsum[w]; wsum[w] = run; run += c; }
    wsum[kPshWarps] = run;
  }
  __syncthreads();
  uint32_t ex = wsum[warp] + inc - v;
  *tot = wsum[kPshWarps];
  __syncthreads();
  return ex;
}

__device__ __forceinline__ uint32_t scene_tiles(const PshArgs &a, uint32_t scene) {
  uint32_t start = scene ? a.batch_sep[scene - 1] : 0u;
  uint32_t end = min(a.batch_sep[scene], a.total_N);
  uint32_t n = end > start ? end - start : 0u;
  return (n + a.tile - 1) / a.tile;
}

// ---------------------------------------------------------------------------------------------------------
// Scan of one round's tile table: a warp owns one (scene, bucket) column, turns the per-tile counts into exclusive
// prefixes over the scene's tiles in place (32 tiles per step, warp shuffle scan) and writes the column total.
// which = 0: round A (totals -> count0, kept), 1: round B attempts (-> attB), 2: round C movers (-> movC).
__global__ void __launch_bounds__(kPshThreads) psh_scan_kernel(PshArgs a, int which) {
  const int lane = threadIdx.x & 31;
  const uint32_t col_lin = blockIdx.x * kPshWarps + (threadIdx.x >> 5);
  if (col_lin >= a.batch * a.nbp) return;
  const uint32_t scene = col_lin / a.nbp, col = col_lin % a.nbp;
  const uint32_t tiles = scene_tiles(a, scene);
  uint32_t *tab = (which == 0 ? a.tabA : (which == 1 ? a.tabB : a.tabC)) + tab_at(a, scene, col, 0);
  uint32_t run = 0;
  for (uint32_t t0 = 0; t0 < tiles; t0 += 32) {
    const uint32_t t = t0 + lane;
    const uint32_t v = t < tiles ? tab[t] : 0u;
    uint32_t inc = v;
#pragma unroll
    for (int d = 1; d < 32; d <<= 1) {
      const uint32_t o = __shfl_up_sync(0xFFFFFFFFu, inc, d);
      if (lane >= d) inc += o;
    }
    if (t < tiles) tab[t] = run + inc - v;
    run += __shfl_sync(0xFFFFFFFFu, inc, 31);
  }
  if (lane == 0) {
    if (which == 0) {
      a.count0[col_lin] = run;
      a.kept[col_lin] = (col == kRecycleBucket) ? run : min(run, a.cap);
    } else if (which == 1) {
      a.attB[col_lin] = run;
    } else {
      a.movC[col_lin] = run;
    }
  }
}

// ---------------------------------------------------------------------------------------------------------
// K3: round A ranks, overflow detection, probe walk, round B histogram
__global__ void __launch_bounds__(kPshThreads) psh_rankA_kernel(PshArgs a) {
  extern __shared__ __align__(16) unsigned char smem_raw[];
  __shared__ uint32_t pending_cnt;
  TileSmem s = carve(smem_raw, a.nbp, a.tile);
  TileInfo t = tile_info(a);
  if (!t.live) return;
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  zero_whist(s, a.nbp);
  // rank base of this tile (the scanned round A table) and the scene's kept counts: requested first, so that their
  // latency runs under the counting sweep
  const uint32_t so = t.scene * a.nbp;
  for (uint32_t b = threadIdx.x; b < a.nbp; b += kPshThreads) {
    s.aux4[b] = 0;
    s.tbase[b] = a.tabA[tab_at(a, t.scene, b, t.tile)];
    s.aux[b] = a.kept[so + b];
  }
  if (threadIdx.x == 0) pending_cnt = 0;
  __syncthreads();
  AxisScale ax[3];
  load_axes(a, ax);
  const HashPlan hp = make_hash_plan(a.hash_type, a.divisor, a.nb);
  const float ratio = probe_ratio(a.num_vox, a.divisor);
  // LCG jump constants of this lane for the warp-wide phase of the walk: probe kSoloProbes + 32 j + lane uses the
  // stream state n = 32 j + lane + 1 steps after the solo probes, s_n = A^n s_0 + C_n (mod 2^32), C_n = c (A^(n-1) + ... + 1)
  constexpr uint32_t kSoloProbes = 8;
  constexpr uint32_t kWarpBatches = (kNumProbes - kSoloProbes + 31) / 32;
  uint32_t jump_a[kWarpBatches], jump_c[kWarpBatches];
#pragma unroll
  for (uint32_t j = 0; j < kWarpBatches; ++j) {
    jump_a[j] = g_lcg_jumps.a[j * 32 + lane];      // n = 32 j + lane + 1 steps
    jump_c[j] = g_lcg_jumps.c[j * 32 + lane];
  }
  const uint32_t wt = a.tile / kPshWarps;
  const uint32_t w0 = warp * wt, w1 = min(w0 + wt, t.cnt);
  uint16_t *st = s.stage + warp * kStageHalves;
  uint16_t *wh = s.whist + warp * a.nbp;
  // sweep 1: the keys kernel 1 left in scratch (a whole group of loads in flight) and per-warp counts
  const uint16_t *gkeys = a.keys + t.start + t.t0;
  for (uint32_t g = w0; g < w1; g += kGroup) {
    uint32_t gc = min(kGroup, w1 - g);
    constexpr int kBatches = kGroup / 32;
    uint32_t kk[kBatches];
#pragma unroll
    for (int u = 0; u < kBatches; ++u) {
      const uint32_t k = u * 32 + lane;
      kk[u] = k < gc ? (uint32_t)gkeys[g + k] : 0u;
    }
#pragma unroll
    for (int u = 0; u < kBatches; ++u) {
      if ((uint32_t)u * 32 >= gc) break;
      const uint32_t k = u * 32 + lane;
      const bool valid = k < gc;
      if (valid) s.keys[g + k] = (uint16_t)kk[u];
      warp_count(wh, kk[u], valid, lane);
    }
  }
  __syncthreads();
  warp_prefix(s, a.nbp);
  __syncthreads();
  // sweep 2: ranks; overflowing points choose their attempt bucket and are counted into this tile's round B
  // histogram in shared memory; the tile owns its word of every column of the round B table and writes the non-zero
  // ones with plain stores at the end (the table was zeroed by the host memset).
  uint32_t my_pending = 0;
  for (uint32_t g = w0; g < w1; g += kGroup) {
    uint32_t gc = min(kGroup, w1 - g);
    bool need_coords = false;
    // ranks first (cheap), then stage coordinates only if some lane of the group overflows
    for (uint32_t it = 0; it < gc; it += 32) {
      uint32_t k = it + lane;
      bool valid = k < gc;
      uint32_t key = valid ? s.keys[g + k] : 0u;
      uint32_t rank = warp_rank(wh, s.tbase, key, valid, lane);
      uint32_t gi = t.start + t.t0 + g + k;
      bool over = valid && key != kRecycleBucket && rank >= a.cap;
      if (valid && !over) {
        a.bucket_id[gi] = (uint16_t)key;
        a.bucket_offset[gi] = rank;
        if (key == kRecycleBucket && rank >= a.cap && a.nb > 1) ++my_pending;
      }
      if (valid && over) s.keys[g + k] = (uint16_t)(0x8000u | key);   // mark for the walk below
      need_coords |= (__any_sync(0xFFFFFFFFu, over) != 0);
    }
    if (!need_coords) continue;
    uint32_t skew = warp_stage(a, t.start + t.t0 + g, gc, st, lane);
    // Walk in two phases.  Phase 1: every overflowing point tries its first kSoloProbes probes on its own lane
    // (scenes with free buckets nearby resolve almost everything here, 32 points at a time).  Phase 2: a point
    // that is still unresolved gets the whole warp: lane l evaluates probe kSoloProbes + 32 j + l of batch j (its
    // position in the point's LCG streams is reached by a jump, s_n = A^n s_0 + C_n), and the first admissible
    // probe in table order is the lowest lane of the first batch that has one, so long walks (LiDAR scans at 90 %
    // load) no longer hold the other 31 lanes up.
    for (uint32_t it = 0; it < gc; it += 32) {
      uint32_t k = it + lane;
      bool valid = k < gc;
      uint32_t mk = valid ? s.keys[g + k] : 0u;
      const bool marked = valid && (mk & 0x8000u);
      const uint32_t init = mk & 0x7FFFu;
      uint32_t vox[3] = {0u, 0u, 0u};
      ProbeStream ps{};
      const uint32_t pt = t.t0 + g + k;
      uint32_t found = a.nb;                           // a.nb = "no admissible probe" column
      bool open = marked;
      if (marked) {
        load_vox(st, skew, k, ax, vox);
        probe_stream_init(a.key, t.scene + a.scene_base, pt, ps);
        uint32_t r[4], nvox[3];
        for (uint32_t p = 0; p < kSoloProbes; ++p) {
          probe_stream_next(ps, r);
          perturb_vox(r, a.num_vox, ratio, a.probe + 3u * p, vox, nvox);
          const uint32_t c = first_hash(hp, nvox[0], nvox[1], nvox[2]);
          if (c != init && c != kRecycleBucket && s.aux[c] < a.cap) { found = c; open = false; break; }
        }
      }
      uint32_t todo = __ballot_sync(0xFFFFFFFFu, open);
      while (todo) {
        const int src = __ffs(todo) - 1;
        todo &= todo - 1;
        uint32_t bvox[3], bs[4];
#pragma unroll
        for (int d = 0; d < 3; ++d) bvox[d] = __shfl_sync(0xFFFFFFFFu, vox[d], src);
#pragma unroll
        for (int q = 0; q < 4; ++q) bs[q] = __shfl_sync(0xFFFFFFFFu, ps.s[q], src);   // state after the solo probes
        const uint32_t binit = __shfl_sync(0xFFFFFFFFu, init, src);
#pragma unroll
        for (uint32_t j = 0; j < kWarpBatches; ++j) {
          const uint32_t p = kSoloProbes + j * 32 + lane;
          uint32_t r[4], nvox[3];
#pragma unroll
          for (int q = 0; q < 4; ++q) {
            const uint32_t sv = bs[q] * jump_a[j] + jump_c[j];
            r[q] = sv ^ (sv >> 15);
          }
          bool ok = false;
          uint32_t c = 0;
          if (p < kNumProbes) {
            perturb_vox(r, a.num_vox, ratio, a.probe + 3u * p, bvox, nvox);
            c = first_hash(hp, nvox[0], nvox[1], nvox[2]);
            ok = c != binit && c != kRecycleBucket && s.aux[c] < a.cap;
          }
          const uint32_t hit = __ballot_sync(0xFFFFFFFFu, ok);
          if (hit) {
            const uint32_t tc = __shfl_sync(0xFFFFFFFFu, c, __ffs(hit) - 1);
            if (lane == src) found = tc;
            break;
          }
        }
      }
      if (marked) {
        uint32_t gi = t.start + pt;
        a.bucket_id[gi] = (uint16_t)found;
        a.bucket_offset[gi] = kPending;
        atomicAdd(&s.aux4[found], 1u);
        ++my_pending;
      }
    }
  }
  if (my_pending) atomicAdd(&pending_cnt, my_pending);
  __syncthreads();
  if (threadIdx.x == 0) a.tile_pending[t.row] = pending_cnt;
  if (pending_cnt)
    for (uint32_t b = threadIdx.x; b < a.nbp; b += kPshThreads) {
      const uint32_t c = s.aux4[b];
      if (c) a.tabB[tab_at(a, t.scene, b, t.tile)] = c;
    }
}

// ---------------------------------------------------------------------------------------------------------
// K5: resolve round B, choose round C targets, round C histogram
__global__ void __launch_bounds__(kPshThreads) psh_resolveB_kernel(PshArgs a) {
  extern __shared__ __align__(16) unsigned char smem_raw[];
  __shared__ uint32_t mover_cnt;
  __shared__ uint32_t wsum[kPshWarps + 1];
  TileSmem s = carve(smem_raw, a.nbp, a.tile);
  TileInfo t = tile_info(a);
  if (!t.live) return;
  const bool pending = a.tile_pending[t.row] != 0;
  if (!pending && t.tile != 0) {
    if (threadIdx.x == 0) a.tile_movers[t.row] = 0;
    return;                       // this tile's round C row stays zero (host memset)
  }
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const uint32_t so = t.scene * a.nbp;
  // Round B totals of the scene from the attempt table: rank base of this tile (tbase), free capacity (aux),
  // kept count (aux2), recycle offset of the first rejected attempt per bucket (aux3).  The tile-0 CTA also
  // publishes the bucket counts after round B.
  {
    uint32_t carry = 0;
    for (uint32_t b0 = 0; b0 < a.nbp; b0 += kPshThreads) {
      const uint32_t b = b0 + threadIdx.x;
      uint32_t rej = 0;
      if (b < a.nbp) {
        const uint32_t pre = a.tabB[tab_at(a, t.scene, b, t.tile)], att = a.attB[so + b];
        const uint32_t kept = a.kept[so + b];
        const uint32_t fr = (b != kRecycleBucket && b < a.nb && kept < a.cap) ? a.cap - kept : 0u;
        const uint32_t acc = min(att, fr);
        rej = att - acc;
        s.tbase[b] = pre; s.aux[b] = fr; s.aux2[b] = kept;
        if (t.tile == 0 && b != kRecycleBucket) a.cntB[so + b] = kept + acc;
      }
      uint32_t tot;
      const uint32_t ex = block_excl_scan(rej, wsum, &tot);
      if (b < a.nbp) s.aux3[b] = carry + ex;
      carry += tot;
    }
    if (t.tile == 0 && threadIdx.x == 0) a.cntB[so + kRecycleBucket] = a.count0[so + kRecycleBucket] + carry;
  }
  if (!pending) {
    if (threadIdx.x == 0) a.tile_movers[t.row] = 0;
    return;
  }
  zero_whist(s, a.nbp);
  for (uint32_t b = threadIdx.x; b < a.nbp; b += kPshThreads) s.aux4[b] = 0;
  if (threadIdx.x == 0) mover_cnt = 0;
  __syncthreads();
  const uint32_t wt = a.tile / kPshWarps;
  const uint32_t w0 = warp * wt, w1 = min(w0 + wt, t.cnt);
  uint16_t *wh = s.whist + warp * a.nbp;
  const uint32_t gbase = t.start + t.t0;
  // keys of pending points; 0xFFFE marks a settled recycle-bucket point beyond the capacity (a round C mover),
  // 0xFFFF any other settled point, so the second sweep does not have to read ids and offsets again.  Four
  // batches of loads are in flight per warp.
  for (uint32_t it0 = w0; it0 < w1; it0 += 128) {
    uint32_t offs[4], keys[4];
#pragma unroll
    for (int u = 0; u < 4; ++u) {
      const uint32_t k = it0 + u * 32 + lane;
      offs[u] = 0; keys[u] = 0;
      if (k < w1) { offs[u] = a.bucket_offset[gbase + k]; keys[u] = a.bucket_id[gbase + k]; }
    }
#pragma unroll
    for (int u = 0; u < 4; ++u) {
      const uint32_t k = it0 + u * 32 + lane;
      if (it0 + u * 32 >= w1) break;
      const bool inb = k < w1;
      const bool valid = inb && offs[u] == kPending;
      if (inb) {
        const bool over = keys[u] == kRecycleBucket && offs[u] >= a.cap && a.nb > 1;
        s.keys[k] = valid ? (uint16_t)keys[u] : (over ? (uint16_t)0xFFFEu : (uint16_t)0xFFFFu);
      }
      warp_count(wh, keys[u], valid, lane);
    }
  }
  __syncthreads();
  warp_prefix(s, a.nbp);
  __syncthreads();
  AxisScale ax[3];
  load_axes(a, ax);
  const HashPlan hp = make_hash_plan(a.hash_type, a.divisor, a.nb);
  const float ratio = probe_ratio(a.num_vox, a.divisor);
  const uint32_t count0_recycle = a.count0[so + kRecycleBucket];
  uint32_t my_movers = 0;
  for (uint32_t it = w0; it < w1; it += 32) {
    uint32_t k = it + lane;
    bool inb = k < w1;
    uint32_t kk = inb ? s.keys[k] : 0xFFFFu;
    bool valid = inb && kk < 0xFFFEu;
    uint32_t q = warp_rank(wh, s.tbase, kk, valid, lane);
    if (!inb) continue;
    uint32_t gi = gbase + k;
    bool mover = false;
    uint32_t recycle_off = 0;
    if (valid) {
      uint32_t fr = s.aux[kk];
      if (q < fr) {
        a.bucket_id[gi] = (uint16_t)kk;
        a.bucket_offset[gi] = s.aux2[kk] + q;
      } else {
        recycle_off = count0_recycle + s.aux3[kk] + (q - fr);
        if (recycle_off < a.cap || a.nb <= 1) {
          a.bucket_id[gi] = (uint16_t)kRecycleBucket;
          a.bucket_offset[gi] = recycle_off;
        } else {
          mover = true;
        }
      }
    } else {
      mover = kk == 0xFFFEu;
    }
    if (mover) {
      uint32_t pt = t.t0 + k;
      uint32_t vox[3], nvox[3], r[4];
#pragma unroll
      for (int d = 0; d < 3; ++d) vox[d] = vox_axis(__half2float(a.coord[(size_t)gi * 3 + d]), ax[d]);
      psh_rand(a.key, t.scene + a.scene_base, pt, 128u, r);
      uint32_t p = r[0] % kNumProbes;
      psh_rand(a.key, t.scene + a.scene_base, pt, 129u, r);
      perturb_vox(r, a.num_vox, ratio, a.probe + 3u * p, vox, nvox);
      uint32_t c = first_hash(hp, nvox[0], nvox[1], nvox[2]);
      if (c == kRecycleBucket) {
        psh_rand(a.key, t.scene + a.scene_base, pt, 130u, r);
        c = 1u + r[0] % (a.nb - 1u);
      }
      a.bucket_id[gi] = (uint16_t)c;
      a.bucket_offset[gi] = kPending;
      atomicAdd(&s.aux4[c], 1u);
      ++my_movers;
    }
  }
  if (my_movers) atomicAdd(&mover_cnt, my_movers);
  __syncthreads();
  if (threadIdx.x == 0) a.tile_movers[t.row] = mover_cnt;
  if (mover_cnt)
    for (uint32_t b = threadIdx.x; b < a.nbp; b += kPshThreads) {
      const uint32_t c = s.aux4[b];
      if (c) a.tabC[tab_at(a, t.scene, b, t.tile)] = c;
    }
}

// ---------------------------------------------------------------------------------------------------------
// K7: round C ranks, final (id, offset), scatter of the coordinates, tail padding (grid row y == batch)
__global__ void __launch_bounds__(kPshThreads) psh_scatter_kernel(PshArgs a) {
  extern __shared__ __align__(16) unsigned char smem_raw[];
  if (blockIdx.y == a.batch) {
    // tail rows [total_N, pad_to) take the pad value (src/psh/batch_psh_bucket.cuh:538-547)
    uint64_t h0 = (uint64_t)a.total_N * 3ull, h1 = (uint64_t)a.pad_to * 3ull;
    uint64_t per = (uint64_t)a.tile * 3ull;
    uint64_t b0 = h0 + (uint64_t)blockIdx.x * per;
    uint64_t b1 = min(b0 + per, h1);
    uint16_t *dst = reinterpret_cast<uint16_t *>(a.scatter_coord);
    for (uint64_t e = b0 + threadIdx.x; e < b1; e += kPshThreads) dst[e] = a.pad_bits;
    return;
  }
  __shared__ uint32_t wsum[kPshWarps + 1];
  TileSmem s = carve(smem_raw, a.nbp, a.tile);
  TileInfo t = tile_info(a);
  if (!t.live) {
    // an empty scene still reports zero counters
    if (t.tile == 0)
      for (uint32_t b = threadIdx.x; b < a.nb; b += kPshThreads) { a.bucket_counter[t.scene * a.nb + b] = 0; a.cumsum_counter[t.scene * a.nb + b] = 0; }
    return;
  }
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const uint32_t so = t.scene * a.nbp;
  const bool movers = a.tile_movers[t.row] != 0;
  const uint32_t wt = a.tile / kPshWarps;
  const uint32_t w0 = warp * wt, w1 = min(w0 + wt, t.cnt);
  uint16_t *wh = s.whist + warp * a.nbp;
  uint16_t *st = s.stage + warp * kStageHalves;
  const uint32_t gbase = t.start + t.t0;
  // Round C totals of the scene: final bucket sizes, their exclusive cumsum (aux = first row of each bucket inside
  // the scene) and the rank base of this tile's movers (tbase).  The tile-0 CTA writes the two counter outputs.
  {
    uint32_t carry = 0;
    for (uint32_t b0 = 0; b0 < a.nbp; b0 += kPshThreads) {
      const uint32_t b = b0 + threadIdx.x;
      uint32_t fin = 0;
      if (b < a.nbp) {
        const uint32_t pre = a.tabC[tab_at(a, t.scene, b, t.tile)], mv = a.movC[so + b];
        const uint32_t cb = a.cntB[so + b];
        if (b == kRecycleBucket) fin = (a.nb > 1) ? min(cb, a.cap) : cb;
        else if (b < a.nb) fin = cb + mv;
        s.tbase[b] = pre + cb;
      }
      uint32_t tot;
      const uint32_t ex = block_excl_scan(fin, wsum, &tot);
      if (b < a.nb) {
        s.aux[b] = carry + ex;
        if (t.tile == 0) { a.bucket_counter[t.scene * a.nb + b] = fin; a.cumsum_counter[t.scene * a.nb + b] = carry + ex + fin; }
      }
      carry += tot;
    }
  }
  if (movers) {
    zero_whist(s, a.nbp);
    __syncthreads();
    for (uint32_t it = w0; it < w1; it += 32) {
      uint32_t k = it + lane;
      bool inb = k < w1;
      bool valid = false;
      uint32_t key = 0;
      if (inb) {
        key = a.bucket_id[gbase + k];
        valid = a.bucket_offset[gbase + k] == kPending;
      }
      warp_count(wh, key, valid, lane);
    }
    __syncthreads();
    warp_prefix(s, a.nbp);
  }
  __syncthreads();
  uint16_t *dst = reinterpret_cast<uint16_t *>(a.scatter_coord);
  for (uint32_t g = w0; g < w1; g += kGroup) {
    uint32_t gc = min(kGroup, w1 - g);
    uint32_t skew = warp_stage(a, gbase + g, gc, st, lane);
    // ids and offsets of the whole group are requested before the first is used: one batch of loads in flight per
    // warp left this loop waiting on memory latency (issue slots 13 % busy on 8 x 1M points)
    constexpr int kBatches = kGroup / 32;
    uint32_t ids[kBatches], offs[kBatches];
#pragma unroll
    for (int u = 0; u < kBatches; ++u) {
      const uint32_t k = u * 32 + lane;
      ids[u] = 0; offs[u] = 0;
      if (k < gc) { ids[u] = a.bucket_id[gbase + g + k]; offs[u] = a.bucket_offset[gbase + g + k]; }
    }
#pragma unroll
    for (int u = 0; u < kBatches; ++u) {
      const uint32_t it = u * 32;
      if (it >= gc) break;
      uint32_t k = it + lane;
      bool inb = k < gc;
      uint32_t gi = gbase + g + k;
      uint32_t id = ids[u], off = offs[u];
      if (movers) {
        bool valid = inb && off == kPending;
        uint32_t r = warp_rank(wh, s.tbase, id, valid, lane);
        if (valid) { off = r; a.bucket_offset[gi] = off; }
      }
      if (inb) {
        uint64_t row = (uint64_t)t.start + s.aux[id] + off;
        if (row < a.pad_to) {
          // a row is 6 bytes: 4-byte aligned when the row index is even, else at 2 mod 4
          uint16_t *d3 = dst + row * 3ull;
          const uint16_t *s3 = st + skew + 3u * k;
          const uint32_t c0 = s3[0], c1 = s3[1], c2 = s3[2];
          if (!a.out_aligned) {
            d3[0] = (uint16_t)c0; d3[1] = (uint16_t)c1; d3[2] = (uint16_t)c2;
          } else if ((row & 1ull) == 0) {
            *reinterpret_cast<uint32_t *>(d3) = c0 | (c1 << 16);
            d3[2] = (uint16_t)c2;
          } else {
            d3[0] = (uint16_t)c0;
            *reinterpret_cast<uint32_t *>(d3 + 1) = c1 | (c2 << 16);
          }
        }
      }
    }
  }
}

// ---------------------------------------------------------------------------------------------------------
static int psh_validate(uint32_t total_N, uint32_t batch, uint32_t num_bucket, uint32_t divisor, uint32_t cap,
                        uint32_t num_vox, uint32_t pad_to, uint32_t hash_type) {
  if (batch == 0) return set_error(F3D_ERR_ARG, "batch_sep is empty");
  if (divisor == 0 || num_bucket == 0 || cap == 0 || num_vox == 0)
    return set_error(F3D_ERR_ARG, "num_bucket, bucket_divisor, bucket_size and num_vox must be positive");
  if (num_vox / divisor > num_bucket) return set_error(F3D_ERR_ARG, "bucket divisor too small");
  if (pad_to < total_N)
    return set_error(F3D_ERR_ARG, "Output coord buffer length(%u) is smaller than the input length(%u).", pad_to, total_N);
  if (hash_type < 1 || hash_type > 4)
    return set_error(F3D_ERR_ARG, "Currently only four types of hash modes are supported. Requested hash_type=%u is unsupported.", hash_type);
  if (num_bucket > 0x7FFEu) return set_error(F3D_ERR_ARG, "num_bucket=%u exceeds the supported 32766", num_bucket);
  if (num_vox > 0x10000u) return set_error(F3D_ERR_ARG, "num_vox=%u exceeds the 16-bit voxel range", num_vox);
  return F3D_OK;
}

struct PshPlan { uint32_t tile, tiles_max, nbp; size_t scratch_words; size_t smem_hist, smem_rank; };

// Scratch of one call in 32-bit words: three tile tables, five per-scene tables, two per-tile flags, the 16-bit keys.
static size_t psh_scratch_words(uint32_t batch, uint32_t tiles_max, uint32_t nbp, uint32_t total_n) {
  const size_t rows = (size_t)batch * tiles_max;
  return 3 * rows * nbp + 5 * (size_t)batch * nbp + 2 * rows + ((size_t)total_n + 1) / 2;
}

// Tiles of 2048 points.  A batch that gives fewer tiles than the GPU has SMs (a single small scan) takes smaller tiles,
// down to 256 points, so that the probe walks of its points spread over more CTAs; when `max_words` is given (the fixed
// scratch of the allocation-free entry point) the tile doubles, up to 16384 points, until the tables fit.  The outputs do
// not depend on the tile size.
static PshPlan psh_plan(uint32_t batch, uint32_t max_n, uint32_t nb, uint32_t total_n, size_t max_words = 0) {
  PshPlan p;
  p.nbp = nb + 1;
  auto set = [&](uint32_t tile) {
    p.tile = tile;
    p.tiles_max = max_n ? (max_n + tile - 1) / tile : 1;
    if (p.tiles_max == 0) p.tiles_max = 1;
    p.scratch_words = psh_scratch_words(batch, p.tiles_max, p.nbp, total_n);
  };
  uint32_t tile = kDefaultTile;
  set(tile);
  while (tile > kMinTile && (size_t)batch * p.tiles_max < kFewTiles) {
    set(tile / 2);
    if (max_words != 0 && p.scratch_words > max_words) { set(tile); break; }
    tile /= 2;
  }
  while (max_words != 0 && p.scratch_words > max_words && tile < kMaxTile) {
    tile *= 2;
    set(tile);
  }
  p.smem_hist = tile_smem_bytes(p.nbp, 0);
  p.smem_rank = tile_smem_bytes(p.nbp, p.tile);
  return p;
}

static int psh_run(PshArgs a, const PshPlan &p, uint32_t *scratch, uint32_t max_n, cudaStream_t st) {
  size_t rows = (size_t)a.batch * p.tiles_max;
  uint32_t *w = scratch;
  a.tabA = w; w += rows * p.nbp;
  a.tabB = w; w += rows * p.nbp;
  a.tabC = w; w += rows * p.nbp;
  a.count0 = w; w += (size_t)a.batch * p.nbp;
  a.kept = w; w += (size_t)a.batch * p.nbp;
  a.cntB = w; w += (size_t)a.batch * p.nbp;
  a.attB = w; w += (size_t)a.batch * p.nbp;
  a.movC = w; w += (size_t)a.batch * p.nbp;
  a.tile_pending = w; w += rows;
  a.tile_movers = w; w += rows;
  a.keys = reinterpret_cast<uint16_t *>(w);
  a.tile = p.tile; a.tiles_max = p.tiles_max; a.nbp = p.nbp;

  int dev = 0;
  cudaGetDevice(&dev);
  // opt in once per device to the large dynamic shared memory the rank kernels may ask for
  F3D_TRY(ensure_dynamic_smem(reinterpret_cast<const void *>(psh_hist_kernel), dev, 200 * 1024));
  F3D_TRY(ensure_dynamic_smem(reinterpret_cast<const void *>(psh_rankA_kernel), dev, 200 * 1024));
  F3D_TRY(ensure_dynamic_smem(reinterpret_cast<const void *>(psh_resolveB_kernel), dev, 200 * 1024));
  F3D_TRY(ensure_dynamic_smem(reinterpret_cast<const void *>(psh_scatter_kernel), dev, 200 * 1024));
  if (p.smem_rank > 200 * 1024) return set_error(F3D_ERR_UNSUPPORTED, "num_bucket=%u needs %zu bytes of shared memory", a.nb, p.smem_rank);

  dim3 grid(p.tiles_max, a.batch);
  const unsigned scan_blocks = (unsigned)(((size_t)a.batch * p.nbp + kPshWarps - 1) / kPshWarps);
  // the round A table is fully rewritten by the histogram kernel for live tiles; the round B and C tables are
  // accumulated with atomics and must start at zero (they are adjacent: one memset)
  if (max_n > 0) {
    F3D_CUDA_TRY(cudaMemsetAsync(a.tabB, 0, 2 * rows * p.nbp * sizeof(uint32_t), st));
    psh_hist_kernel<<<grid, kPshThreads, p.smem_hist, st>>>(a);
    psh_scan_kernel<<<scan_blocks, kPshThreads, 0, st>>>(a, 0);
    psh_rankA_kernel<<<grid, kPshThreads, p.smem_rank, st>>>(a);
    psh_scan_kernel<<<scan_blocks, kPshThreads, 0, st>>>(a, 1);
    psh_resolveB_kernel<<<grid, kPshThreads, p.smem_rank, st>>>(a);
    psh_scan_kernel<<<scan_blocks, kPshThreads, 0, st>>>(a, 2);
  } else {
    F3D_CUDA_TRY(cudaMemsetAsync(a.bucket_counter, 0, (size_t)a.batch * a.nb * 4, st));
    F3D_CUDA_TRY(cudaMemsetAsync(a.cumsum_counter, 0, (size_t)a.batch * a.nb * 4, st));
  }
  uint32_t pad_rows = a.pad_to - a.total_N;
  uint32_t gx = max_n ? p.tiles_max : 0;
  uint32_t pad_blocks = (pad_rows + p.tile - 1) / p.tile;
  if (pad_blocks > gx) gx = pad_blocks;
  if (gx > 0) {
    dim3 grid2(gx, a.batch + 1);
    a.tiles_max = p.tiles_max;
    psh_scatter_kernel<<<grid2, kPshThreads, p.smem_rank, st>>>(a);
  }
  return check_launch("psh kernels", (max_n > 0 ? 6 : 0) + (gx > 0 ? 1 : 0));
}

// The kernel arguments of one PSH call from the C-ABI arguments (shared by the two entry points below).
static PshArgs psh_pack_args(
    const void *coord, void *bucket_id, void *bucket_counter, void *bucket_offset, const void *batch_sep,
    uint32_t total_N, uint32_t batch_size, uint32_t num_bucket, uint32_t bucket_divisor, uint32_t bucket_size,
    uint32_t num_vox, const void *bbox_min, const void *bbox_max, const void *probe_offsets, void *cumsum_counter,
    void *scatter_coord, uint32_t pad_to_N, float pad_num, uint32_t hash_type) {
  PshArgs a{};
  a.coord = static_cast<const __half *>(coord);
  a.bucket_id = static_cast<uint16_t *>(bucket_id);
  a.bucket_counter = static_cast<uint32_t *>(bucket_counter);
  a.bucket_offset = static_cast<uint32_t *>(bucket_offset);
  a.batch_sep = static_cast<const uint32_t *>(batch_sep);
  a.cumsum_counter = static_cast<uint32_t *>(cumsum_counter);
  a.scatter_coord = static_cast<__half *>(scatter_coord);
  a.bbox_min = static_cast<const __half *>(bbox_min);
  a.bbox_max = static_cast<const __half *>(bbox_max);
  a.probe = static_cast<const int16_t *>(probe_offsets);
  a.total_N = total_N; a.batch = batch_size; a.nb = num_bucket; a.divisor = bucket_divisor; a.cap = bucket_size;
  a.num_vox = num_vox; a.hash_type = hash_type; a.pad_to = pad_to_N;
  a.pad_bits = __half_as_ushort(__float2half_rn(pad_num));
  a.coord_aligned = (reinterpret_cast<uintptr_t>(coord) % 16 == 0) ? 1 : 0;
  a.out_aligned = (reinterpret_cast<uintptr_t>(scatter_coord) % 4 == 0) ? 1 : 0;
  uint64_t sd = f3d::seed();
  a.key.k0 = (uint32_t)sd; a.key.k1 = (uint32_t)(sd >> 32);
  a.scene_base = f3d::scene_base();
  return a;
}

}  // namespace f3d

using namespace f3d;

extern "C" int f3d_batch_psh_scatter_pad_hash(
    const void *coord, void *bucket_id, void *bucket_counter, void *bucket_offset, const void *batch_sep,
    uint32_t total_N, uint32_t batch_size, uint32_t instance_max_N, uint32_t num_bucket, uint32_t bucket_divisor,
    uint32_t bucket_size, uint32_t num_vox, const void *bbox_min, const void *bbox_max, const void *probe_offsets,
    void *cumsum_counter, void *scatter_coord, uint32_t pad_to_N, float pad_num, uint32_t hash_type,
    int device, void *stream) {
  F3D_TRY(psh_validate(total_N, batch_size, num_bucket, bucket_divisor, bucket_size, num_vox, pad_to_N, hash_type));
  DeviceGuard guard(device);
  cudaStream_t st = reinterpret_cast<cudaStream_t>(stream);
  if (instance_max_N > total_N) instance_max_N = total_N;
  PshPlan p = psh_plan(batch_size, instance_max_N, num_bucket, total_N);
  void *scratch = nullptr;
  F3D_TRY(workspace(device, 0, p.scratch_words * sizeof(uint32_t), st, &scratch));
  PshArgs a = psh_pack_args(coord, bucket_id, bucket_counter, bucket_offset, batch_sep, total_N, batch_size, num_bucket,
                            bucket_divisor, bucket_size, num_vox, bbox_min, bbox_max, probe_offsets, cumsum_counter,
                            scatter_coord, pad_to_N, pad_num, hash_type);
  F3D_TRY(maybe_sync(st, "batch_psh_scatter_pad_hash"));
  F3D_TRY(psh_run(a, p, static_cast<uint32_t *>(scratch), instance_max_N, st));
  return maybe_sync(st, "batch_psh_scatter_pad_hash");
}


// ---------------------------------------------------------------------------------------------------------
// Variant for callers that must not allocate device memory.
//
// Some hosts of this library cannot call cudaMalloc at all: a serving runtime that has handed every byte of the
// GPU to its own arena (a stray cudaMalloc then fails or is treated as a bug), or a latency-critical loop that
// cannot afford the device-wide synchronisation cudaMalloc and cudaFree imply.  For them the tile tables and
// per-scene counters of the three ranking rounds live in the fixed array below instead of the grow-on-demand
// workspace.  Every GPU that loads the library holds these 4 MiB until the process exits.
//
// The array is shared by all calls and keeps the previous call's contents; the tables that are accumulated
// with atomics are cleared on the caller's stream at the start of every call, everything else is rewritten
// before it is read.  Two calls that overlap on the same GPU (different streams or threads) race on it.
constexpr size_t kStaticScratchWords = size_t(1) << 20;       // 4 MiB
static __device__ __align__(256) uint32_t g_psh_static_scratch[kStaticScratchWords];

namespace f3d {
// The symbol name above is only a host-side handle; kernels need the device address, looked up once per
// device with that device current.
static int static_scratch_ptr(int device, uint32_t **out) {
  static std::mutex mu;
  static std::map<int, uint32_t *> ptrs;
  if (device < 0) return set_error(F3D_ERR_ARG, "device %d out of range", device);
  std::lock_guard<std::mutex> lk(mu);
  auto it = ptrs.find(device);
  if (it == ptrs.end()) {
    void *p = nullptr;
    cudaError_t e = cudaGetSymbolAddress(&p, g_psh_static_scratch);
    if (e != cudaSuccess) return set_error(F3D_ERR_CUDA, "cudaGetSymbolAddress(static scratch): %s", cudaGetErrorString(e));
    it = ptrs.emplace(device, static_cast<uint32_t *>(p)).first;
  }
  *out = it->second;
  return F3D_OK;
}
}  // namespace f3d

extern "C" int f3d_batch_psh_scatter_pad_hash_noalloc(
    const void *coord, void *bucket_id, void *bucket_counter, void *bucket_offset, const void *batch_sep,
    uint32_t total_N, uint32_t batch_size, uint32_t instance_max_N, uint32_t num_bucket, uint32_t bucket_divisor,
    uint32_t bucket_size, uint32_t num_vox, const void *bbox_min, const void *bbox_max, const void *probe_offsets,
    void *cumsum_counter, void *scatter_coord, uint32_t pad_to_N, float pad_num, uint32_t hash_type,
    int device, void *stream) {
  F3D_TRY(psh_validate(total_N, batch_size, num_bucket, bucket_divisor, bucket_size, num_vox, pad_to_N, hash_type));
  DeviceGuard guard(device);
  cudaStream_t st = reinterpret_cast<cudaStream_t>(stream);
  if (instance_max_N > total_N) instance_max_N = total_N;
  PshPlan p = psh_plan(batch_size, instance_max_N, num_bucket, total_N, kStaticScratchWords);
  if (p.scratch_words > kStaticScratchWords)
    return set_error(F3D_ERR_UNSUPPORTED,
                     "batch_psh_scatter_pad_hash_noalloc: this batch needs %zu scratch words (batch %u x %u tiles x %u "
                     "buckets) but the fixed scratch holds %zu; use batch_psh_scatter_pad_hash or a smaller batch",
                     p.scratch_words, batch_size, p.tiles_max, num_bucket, kStaticScratchWords);
  uint32_t *scratch = nullptr;
  F3D_TRY(static_scratch_ptr(device, &scratch));
  PshArgs a = psh_pack_args(coord, bucket_id, bucket_counter, bucket_offset, batch_sep, total_N, batch_size, num_bucket,
                            bucket_divisor, bucket_size, num_vox, bbox_min, bbox_max, probe_offsets, cumsum_counter,
                            scatter_coord, pad_to_N, pad_num, hash_type);
  // the sync_stream debug switch is honoured like in the regular entry point (a stream synchronisation allocates nothing)
  F3D_TRY(maybe_sync(st, "batch_psh_scatter_pad_hash_noalloc"));
  F3D_TRY(psh_run(a, p, scratch, instance_max_N, st));
  return maybe_sync(st, "batch_psh_scatter_pad_hash_noalloc");
}
