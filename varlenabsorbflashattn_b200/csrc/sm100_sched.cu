// Single-CTA scheduler kernel: see sm100_sched.cuh.
#include "sm100_sched.cuh"
#include "profile.cuh"

namespace vafa {
namespace {

constexpr int kSchedThreads = 1024;
constexpr int kBuckets = 512;

struct Unit {
  int o_start, o_rows, i_start, i_len, diag, masked;
};

// Visit every 128-row outer tile of every segment.  f(unit) is called by the owning thread.
template <typename F>
__device__ __forceinline__ void for_each_unit(const SchedParams& p, F f) {
  for (int s = threadIdx.x; s < p.n_seg; s += kSchedThreads) {
    const int q0 = p.cu_q[s], Lq = p.cu_q[s + 1] - q0;
    const int k0 = p.cu_k[s], Lk = p.cu_k[s + 1] - k0;
    const int off = Lk - Lq;
    if (p.mode == kSchedDkv) {
      for (int j0 = 0; j0 < Lk; j0 += kTile) {
        Unit u;
        u.o_start = k0 + j0;
        u.o_rows = min(kTile, Lk - j0);
        int ibeg = 0;
        if (p.causal) ibeg = max(0, j0 - off);
        u.i_len = max(0, Lq - ibeg);
        u.i_start = q0 + ibeg;
        u.diag = j0 - off - ibeg;   // key row r of the tile and inner row ii: visible iff ii >= r + diag
        u.masked = p.causal;
        f(u);
      }
    } else {
      for (int i0 = 0; i0 < Lq; i0 += p.tile_rows) {
        Unit u;
        u.o_start = q0 + i0;
        u.o_rows = min(p.tile_rows, Lq - i0);
        int kend = Lk;
        if (p.causal) kend = min(Lk, i0 + u.o_rows + off);
        u.i_len = max(0, kend);
        u.i_start = k0;
        u.diag = i0 + off;          // query row r of the tile sees inner row jj iff jj <= r + diag
        u.masked = p.causal;
        f(u);
      }
    }
  }
}

__device__ __forceinline__ int n_blocks(int len) { return (len + kTile - 1) / kTile; }

__global__ void __launch_bounds__(kSchedThreads) sched_kernel(SchedParams p) {
  __shared__ int s_hist[kBuckets];
  __shared__ int s_units, s_blocks, s_items, s_rows, s_bs, s_combine;

  if (threadIdx.x == 0) { s_units = 0; s_blocks = 0; s_combine = 0; }
  for (int b = threadIdx.x; b < kBuckets; b += kSchedThreads) s_hist[b] = 0;
  __syncthreads();

  // pass 1: totals
  {
    int units = 0, blocks = 0;
    for_each_unit(p, [&](const Unit& u) {
      if (u.i_len > 0) { units += 1; blocks += n_blocks(u.i_len); }
    });
    if (units) { atomicAdd(&s_units, units); atomicAdd(&s_blocks, blocks); }
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
          const long long t = ((long long)s_blocks * p.H + 2LL * p.sm_count - 1) / (2LL * p.sm_count);
          bs = (int)max(8LL, t);
        }
      }
    }
    s_bs = bs;
  }
  __syncthreads();

  // pass 2: make the split fit the capacities (double the slice until it does)
  for (int round = 0; round < 24; ++round) {
    if (threadIdx.x == 0) { s_items = 0; s_rows = 0; }
    __syncthreads();
    const int bs = s_bs;
    int items = 0, rows = 0;
    for_each_unit(p, [&](const Unit& u) {
      const int nb = n_blocks(u.i_len);
      const int ns = (bs > 0 && nb > bs) ? (nb + bs - 1) / bs : 1;
      items += ns;
      if (ns > 1) rows += ns * u.o_rows;
    });
    if (items) atomicAdd(&s_items, items);
    if (rows) atomicAdd(&s_rows, rows);
    __syncthreads();
    const bool fits = (s_items <= p.cap_items) && (s_rows <= p.cap_rows);
    __syncthreads();
    if (fits || s_bs == 0) break;
    if (threadIdx.x == 0) s_bs = (s_bs >= (1 << 24)) ? 0 : s_bs * 2;
    __syncthreads();
  }
  const int bs = s_bs;

  // pass 3: histogram of item costs
  for_each_unit(p, [&](const Unit& u) {
    const int nb = n_blocks(u.i_len);
    const int ns = (bs > 0 && nb > bs) ? (nb + bs - 1) / bs : 1;
    const int per = (ns > 1) ? (nb + ns - 1) / ns : nb;
    for (int sp = 0; sp < ns; ++sp) {
      const int b0 = sp * per;
      const int cost = min(per, nb - b0);
      atomicAdd(&s_hist[min(max(cost, 0), kBuckets - 1)], 1);
    }
  });
  __syncthreads();
  // descending exclusive scan: bucket b starts after all larger buckets
  if (threadIdx.x == 0) {
    int run = 0;
    for (int b = kBuckets - 1; b >= 0; --b) {
      const int c = s_hist[b];
      s_hist[b] = run;
      run += c;
    }
    s_items = run;
    s_rows = 0;
  }
  __syncthreads();
  const bool overflow = s_items > p.cap_items;

  // pass 4: emit
  if (!overflow) {
    for_each_unit(p, [&](const Unit& u) {
      const int nb = n_blocks(u.i_len);
      const int ns = (bs > 0 && nb > bs) ? (nb + bs - 1) / bs : 1;
      const int per = (ns > 1) ? (nb + ns - 1) / ns : nb;
      int base = -1;
      if (ns > 1) {
        base = atomicAdd(&s_rows, ns * u.o_rows);
        const int c = atomicAdd(&s_combine, 1);
        CombineUnit cu;
        cu.q_start = u.o_start; cu.q_rows = u.o_rows; cu.base = base; cu.n_splits = ns;
        p.combine[c] = cu;
      }
      for (int sp = 0; sp < ns; ++sp) {
        const int b0 = sp * per;
        const int cost = min(per, nb - b0);
        const int pos = atomicAdd(&s_hist[min(max(cost, 0), kBuckets - 1)], 1);
        WorkItem w;
        w.o_start = u.o_start;
        w.o_rows = u.o_rows;
        w.i_start = u.i_start + b0 * kTile;
        w.i_len = max(0, min(u.i_len - b0 * kTile, per * kTile));
        w.diag = u.diag - b0 * kTile;
        w.masked = u.masked;
        w.partial = (ns > 1) ? base + sp * u.o_rows : -1;
        w.cost = cost;
        p.items[pos] = w;
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

}  // namespace

int launch_scheduler(const SchedParams& p, cudaStream_t s) {
  LaunchScope scope(kKSched, s);
  sched_kernel<<<1, kSchedThreads, 0, s>>>(p);
  VAFA_LAUNCH_CHECK("sched_kernel");
  return 0;
}

}  // namespace vafa
