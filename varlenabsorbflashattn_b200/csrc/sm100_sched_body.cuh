// Body of the single-CTA tile-list builder (see sm100_sched.cuh), as a device function so that it can
// run as CTAs of another kernel's grid as well.  One call = one CTA of kSchedThreads threads.
//
// Order of the emitted work items: segments by descending total cost (bucket sort on a
// logarithmic scale); inside a segment all heads; inside a head the tiles by descending cost and
// their splits.  Persistent CTAs take consecutive items, so the CTAs that run at the same time
// work on tiles of the same (segment, head) and find each other's K/V (or Q/dO) blocks in L2
// instead of each streaming them from HBM, while the large-to-small order keeps the tail short.
#pragma once
#include "sm100_sched.cuh"

namespace vafa {
namespace sched_impl {


constexpr int kSchedThreads = 1024;
constexpr int kBuckets = 512;

struct Seg {
  int q0, Lq, k0, Lk, off;
  int n_tiles;  // outer tiles of the segment
};

struct Unit {
  int o_start, o_rows, i_start, i_len, diag;
};

__device__ __forceinline__ int n_blocks(int len) { return (len + kTile - 1) / kTile; }

__device__ __forceinline__ Seg load_seg(const SchedParams& p, int s) {
  Seg g;
  g.q0 = p.cu_q[s]; g.Lq = p.cu_q[s + 1] - g.q0;
  g.k0 = p.cu_k[s]; g.Lk = p.cu_k[s + 1] - g.k0;
  g.off = g.Lk - g.Lq;
  g.n_tiles = (p.mode == kSchedDkv) ? (g.Lk + kTile - 1) / kTile : (g.Lq + p.tile_rows - 1) / p.tile_rows;
  return g;
}

// Tile t of a segment, t counted in order of descending cost.
__device__ __forceinline__ Unit make_unit(const SchedParams& p, const Seg& g, int t) {
  Unit u;
  if (p.mode == kSchedDkv) {
    // key tiles; under the causal mask the first tiles see the most query rows
    const int j0 = t * kTile;
    u.o_start = g.k0 + j0;
    u.o_rows = min(kTile, g.Lk - j0);
    const int ibeg = p.causal ? max(0, j0 - g.off) : 0;
    u.i_len = max(0, g.Lq - ibeg);
    u.i_start = g.q0 + ibeg;
    u.diag = j0 - g.off - ibeg;  // key row r of the tile and inner row ii: visible iff ii >= r + diag
  } else {
    // query tiles; under the causal mask the last tiles see the most keys
    const int i0 = (p.causal ? (g.n_tiles - 1 - t) : t) * p.tile_rows;
    u.o_start = g.q0 + i0;
    u.o_rows = min(p.tile_rows, g.Lq - i0);
    const int kend = p.causal ? min(g.Lk, i0 + u.o_rows + g.off) : g.Lk;
    u.i_len = max(0, kend);
    u.i_start = g.k0;
    u.diag = i0 + g.off;         // query row r of the tile sees inner row jj iff jj <= r + diag
  }
  return u;
}

__device__ __forceinline__ int n_splits(int nb, int bs) { return (bs > 0 && nb > bs) ? (nb + bs - 1) / bs : 1; }

// Monotone map of a cost to one of kBuckets buckets: 16 buckets per power of two.
__device__ __forceinline__ int cost_bucket(long long c) {
  if (c <= 0) return 0;
  if (c < 16) return (int)c;
  const int lz = __clzll(c);
  const int e = 63 - lz;                                  // floor(log2 c) >= 4
  const int m = (int)((c >> (e - 4)) & 15);               // next four bits
  return min(kBuckets - 1, 16 * (e - 3) + m);
}


// Warp-aggregated histogram add: every lane of the warp calls; the `active` lanes add `v` to hist[bucket]
// and get back the value before their own add.  Lanes that hit the same bucket are served by one atomic
// (a thousand users of equal cost otherwise queue on one shared-memory word); their ranges are
// consecutive in lane order.
__device__ __forceinline__ int warp_hist_add(int* hist, bool active, int bucket, int v) {
  const int lane = threadIdx.x & 31;
  int pos = 0;
  unsigned todo = __ballot_sync(0xffffffffu, active);
  while (todo) {
    const int leader = __ffs(todo) - 1;
    const int b = __shfl_sync(0xffffffffu, bucket, leader);
    const bool mine = active && bucket == b;
    const unsigned same = __ballot_sync(0xffffffffu, mine);
    int incl = mine ? v : 0;
#pragma unroll
    for (int o = 1; o < 32; o <<= 1) {
      const int t = __shfl_up_sync(0xffffffffu, incl, o);
      if (lane >= o) incl += t;
    }
    const int total = __shfl_sync(0xffffffffu, incl, 31);
    int base = 0;
    if (lane == leader) base = atomicAdd(&hist[b], total);
    base = __shfl_sync(0xffffffffu, base, leader);
    if (mine) pos = base + incl - v;
    todo &= ~same;
  }
  return pos;
}

__device__ __forceinline__ long long warp_sum_ll(long long x) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) x += __shfl_xor_sync(0xffffffffu, x, o);
  return x;
}

// Walk all segments with G lanes per segment (G a power of two, 1..32, the same for the whole list):
// lane gl of a group owns tiles gl, gl + G, ... of its segment.  G = 1024 / n_seg rounded up to a power
// of two: few long segments get a whole warp each, a batch of a thousand users one thread each (with a
// warp per one-tile segment the list of 1137 users cost 32 times the instructions).  Every group runs
// the same number of rounds (the body contains warp shuffles); groups past the end get an empty segment.
// Neighbouring groups read neighbouring cu_seqlens entries, so one round costs one memory latency.
// body(g, gl, G)
template <typename F>
__device__ __forceinline__ void for_each_segment(const SchedParams& p, int G, F body) {
  const int per_round = kSchedThreads / G;
  const int gid = threadIdx.x / G, gl = threadIdx.x % G;
  const int rounds = (p.n_seg + per_round - 1) / per_round;
  for (int it = 0; it < rounds; ++it) {
    const int s = it * per_round + gid;
    Seg g = {0, 0, 0, 0, 0, 0};
    if (s < p.n_seg) g = load_seg(p, s);
    body(g, gl, G);
  }
}

__device__ __forceinline__ void sched_build(const SchedParams& p) {
  __shared__ int s_hist[kBuckets];
  __shared__ int s_units, s_items, s_rows, s_bs, s_combine;
  __shared__ unsigned long long s_items64, s_rows64;  // pass 2 counts in 64 bits
  __shared__ long long s_blocks;

  if (threadIdx.x == 0) { s_units = 0; s_blocks = 0; s_combine = 0; }
  for (int b = threadIdx.x; b < kBuckets; b += kSchedThreads) s_hist[b] = 0;
  __syncthreads();

  const int lane = threadIdx.x & 31, wid = threadIdx.x >> 5;
  // lanes per segment (see for_each_segment)
  int G = 1;
  while (G < 32 && G * p.n_seg < kSchedThreads) G <<= 1;

  // pass 1: totals, and the cost histogram for the common case that nothing is split (one item per
  // tile); only a list that does get split goes through passes 2 and 3
  {
    int units = 0;
    long long blocks = 0;
    for_each_segment(p, G, [&](const Seg& g, int t0, int ts) {
      long long cost = 0;
      int items = 0;
      for (int t = t0; t < g.n_tiles; t += ts) {
        const Unit u = make_unit(p, g, t);
        const int nb = n_blocks(u.i_len);
        if (u.i_len > 0) { units += 1; blocks += nb; }
        cost += nb;
        items += 1;
      }
      for (int o = ts >> 1; o > 0; o >>= 1) {
        cost += __shfl_xor_sync(0xffffffffu, cost, o);
        items += __shfl_xor_sync(0xffffffffu, items, o);
      }
      warp_hist_add(s_hist, t0 == 0 && items > 0, cost_bucket(cost), items * p.H);
    });
    units = (int)warp_sum_ll(units);
    blocks = warp_sum_ll(blocks);
    if (lane == 0 && units) { atomicAdd(&s_units, units); atomicAdd((unsigned long long*)&s_blocks, (unsigned long long)blocks); }
  }
  __syncthreads();

  // split policy (forward only): inner blocks per item
  if (threadIdx.x == 0) {
    int bs = 0;  // 0 = never split
    if (p.mode == kSchedFwd) {
      if (p.split_len > 0) {
        bs = p.split_len / kTile;
      } else {
        const long long par = (long long)s_units * p.H;
        if (par > 0 && par < 2LL * p.sm_count) {
          const long long t = (s_blocks * p.H + 2LL * p.sm_count - 1) / (2LL * p.sm_count);
          bs = (int)max(8LL, t);
        }
      }
    }
    s_bs = bs;
  }
  __syncthreads();

  const bool any_split = s_bs != 0;
  if (any_split) {
    for (int b = threadIdx.x; b < kBuckets; b += kSchedThreads) s_hist[b] = 0;
    __syncthreads();
  }
  // pass 2: make the split fit the capacities (double the slice until it does)
  for (int round = 0; any_split && round < 24; ++round) {
    if (threadIdx.x == 0) { s_items64 = 0; s_rows64 = 0; }
    __syncthreads();
    const int bs = s_bs;
    // counted in 64 bits: a short forced slice on very long sequences can pass 2^31 partial rows, and a
    // wrapped 32-bit sum would pass the capacity test below
    long long items = 0, rows = 0;
    for_each_segment(p, G, [&](const Seg& g, int t0, int ts) {
      for (int t = t0; t < g.n_tiles; t += ts) {
        const Unit u = make_unit(p, g, t);
        const int ns = n_splits(n_blocks(u.i_len), bs);
        items += ns;
        if (ns > 1) rows += (long long)ns * u.o_rows;
      }
    });
    items = warp_sum_ll(items);
    rows = warp_sum_ll(rows);
    if (lane == 0 && items) atomicAdd(&s_items64, (unsigned long long)items);
    if (lane == 0 && rows) atomicAdd(&s_rows64, (unsigned long long)rows);
    __syncthreads();
    const bool fits = (s_items64 <= (unsigned long long)p.cap_items / (unsigned long long)p.H) &&
                      (s_rows64 <= (unsigned long long)max(p.cap_rows, 0));
    __syncthreads();
    if (fits || s_bs == 0) break;
    if (threadIdx.x == 0) s_bs = (s_bs >= (1 << 24)) ? 0 : s_bs * 2;
    __syncthreads();
  }
  const int bs = s_bs;

  // pass 3: items per cost bucket of their segment
  if (any_split) for_each_segment(p, G, [&](const Seg& g, int t0, int ts) {
    long long cost = 0;
    int items = 0;
    for (int t = t0; t < g.n_tiles; t += ts) {
      const Unit u = make_unit(p, g, t);
      const int nb = n_blocks(u.i_len);
      cost += nb;
      items += n_splits(nb, bs);
    }
    for (int o = ts >> 1; o > 0; o >>= 1) {
      cost += __shfl_xor_sync(0xffffffffu, cost, o);
      items += __shfl_xor_sync(0xffffffffu, items, o);
    }
    warp_hist_add(s_hist, t0 == 0 && items > 0, cost_bucket(cost), items * p.H);
  });
  __syncthreads();
  // descending exclusive scan: a bucket starts after all buckets of larger cost
  if (wid == 0) {
    // lane j owns buckets [kBuckets - 16 (j+1), kBuckets - 16 j), walked downwards
    constexpr int kPer = kBuckets / 32;
    const int top = kBuckets - 1 - lane * kPer;
    int cnt[kPer], sum = 0;
#pragma unroll
    for (int i = 0; i < kPer; ++i) { cnt[i] = s_hist[top - i]; sum += cnt[i]; }
    int incl = sum;
#pragma unroll
    for (int o = 1; o < 32; o <<= 1) {
      const int v = __shfl_up_sync(0xffffffffu, incl, o);
      if (lane >= o) incl += v;
    }
    int run = incl - sum;  // items in all buckets of larger cost
#pragma unroll
    for (int i = 0; i < kPer; ++i) { s_hist[top - i] = run; run += cnt[i]; }
    if (lane == 31) { s_items = run; s_rows = 0; }
  }
  __syncthreads();
  const bool overflow = s_items > p.cap_items;

  // pass 4: emit, one contiguous range per segment; one warp per segment, lanes over (head, tile)
  if (!overflow) {
    for_each_segment(p, G, [&](const Seg& g, int t0, int ts) {
      int items = 0, pos = 0, n_split_tiles = 0, c0 = 0;
      long long cost = 0;
      for (int t = t0; t < g.n_tiles; t += ts) {
        const int nb = n_blocks(make_unit(p, g, t).i_len);
        const int ns = n_splits(nb, bs);
        cost += nb;
        items += ns;
        n_split_tiles += (ns > 1);
      }
      for (int o = ts >> 1; o > 0; o >>= 1) {
        cost += __shfl_xor_sync(0xffffffffu, cost, o);
        items += __shfl_xor_sync(0xffffffffu, items, o);
        n_split_tiles += __shfl_xor_sync(0xffffffffu, n_split_tiles, o);
      }
      pos = warp_hist_add(s_hist, t0 == 0 && items > 0, cost_bucket(cost), items * p.H);
      if (t0 == 0) {
        if (n_split_tiles) {
          // split-K bookkeeping once per tile: the partial rows are shared by the heads ([row][head])
          c0 = atomicAdd(&s_combine, n_split_tiles);
          int k = 0;
          for (int t = 0; t < g.n_tiles; ++t) {
            const Unit u = make_unit(p, g, t);
            const int ns = n_splits(n_blocks(u.i_len), bs);
            if (ns > 1) {
              CombineUnit cu;
              cu.q_start = u.o_start; cu.q_rows = u.o_rows; cu.n_splits = ns;
              cu.base = atomicAdd(&s_rows, ns * u.o_rows);
              p.combine[c0 + k++] = cu;
            }
          }
        }
      }
      if (ts > 1) {
        // from the group's first lane; the combine units it wrote are read by all lanes below
        pos = __shfl_sync(0xffffffffu, pos, 0, ts);
        c0 = __shfl_sync(0xffffffffu, c0, 0, ts);
        __syncwarp();
      }
      if (items == 0) return;
      if (n_split_tiles == 0) {
        // one item per tile: position is direct
        // lanes over tiles (the unit is computed once), then one store per head
        for (int t = t0; t < g.n_tiles; t += ts) {
          const Unit u = make_unit(p, g, t);
          WorkItem w;
          w.o_start = u.o_start; w.o_rows = u.o_rows; w.i_start = u.i_start; w.i_len = u.i_len;
          w.diag = u.diag; w.masked = p.causal; w.partial = -1;
          for (int h = 0; h < p.H; ++h) {
            w.head = h;
            p.items[pos + h * items + t] = w;
          }
        }
      } else {
        for (int h = t0; h < p.H; h += ts) {
          int at = pos + h * items, k = 0;
          for (int t = 0; t < g.n_tiles; ++t) {
            const Unit u = make_unit(p, g, t);
            const int nb = n_blocks(u.i_len);
            const int ns = n_splits(nb, bs);
            const int per = (ns > 1) ? (nb + ns - 1) / ns : nb;
            const int base = (ns > 1) ? p.combine[c0 + k++].base : -1;
            for (int sp = 0; sp < ns; ++sp) {
              const int b0 = sp * per;
              WorkItem w;
              w.o_start = u.o_start;
              w.o_rows = u.o_rows;
              w.i_start = u.i_start + b0 * kTile;
              w.i_len = max(0, min(u.i_len - b0 * kTile, per * kTile));
              w.diag = u.diag - b0 * kTile;
              w.masked = p.causal;
              w.partial = (ns > 1) ? base + sp * u.o_rows : -1;
              w.head = h;
              p.items[at++] = w;
            }
          }
        }
      }
    });
  }
  __syncthreads();
  if (threadIdx.x == 0) {
    SchedHeader h;
    h.n_items = overflow ? -1 : s_items;
    h.n_combine = s_combine;
    h.n_partial_rows = s_rows;
    h.block_len = bs;
    h.reserved0 = 0;
    h.next_item = 0;
    h.pad[0] = h.pad[1] = 0;
    *p.header = h;
  }
}

}  // namespace sched_impl
}  // namespace vafa
