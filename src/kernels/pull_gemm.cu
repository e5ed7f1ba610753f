// C[M,N] = X[M,K] * W[N,K]^T in bf16 with fp32 accumulation on the 5th-generation tensor
// cores, optionally fused with the pull (all-gather) of W.
//
// Structure of one GEMM CTA (256 threads of which six warps have a role; persistent over
// output tiles):
//   warp 0      TMA producer: loads 128xBK tiles of X and BNxBK tiles of W into a ring of
//               shared-memory stages (128-byte swizzle, mbarrier transaction counts);
//   warp 1      MMA issuer: one thread issues tcgen05.mma (128 x BN x 16 per instruction)
//               from the stages into one of two fp32 accumulators in tensor memory and
//               commits stage-free / accumulator-full mbarriers;
//   warps 2..5  epilogue: tcgen05.ld the finished accumulator (each warp its 32 lanes),
//               convert to bf16 and store to C while the next tile is being multiplied.
//
// Fusion with pull: W lives in the workers' weight buffer of a dense table; each rank holds
// the blocks it owns (published by its push).  Extra "copy" CTAs, placed first in the grid so
// that they never wait behind GEMM CTAs, fetch the remotely owned blocks of W over NVLink
// with plain peer loads, one BN-row panel at a time, and bump a per-panel counter; the TMA
// producer of every GEMM CTA waits for the panel of its current tile (and for nothing
// else), then reads it from local memory with ordinary, non-multicast TMA.  The matrix
// multiply of panel p therefore overlaps the transfer of panels p+1, p+2, ...
//
// The reference has no compute of any kind; the pull it implements (server response plus
// worker-side reassembly, include/ps/kv_app.h:616-717) is what the copy CTAs replace.
//
// Every wait (mbarrier, panel counter) is bounded; on expiry the kernel
// records an error, lets its in-flight copies land, frees its tensor memory and returns.
#include <cuda_bf16.h>

#include <atomic>
#include <cstdlib>
#include <mutex>

#include "ps/device/push_pull.cuh"
#include "ps/device/sm100_ptx.cuh"

namespace psdev {
extern std::atomic<uint64_t> g_launches;

namespace gemm {
using namespace sm100;

constexpr int BM = 128;
constexpr int BK = 64;  // 64 bf16 = 128 bytes = one swizzle row
constexpr int UMMA_K = 16;
constexpr int kThreads = 256;      // warps 0..5: TMA, MMA, 4 x epilogue; warps 6..7: pull ring
constexpr int kCopyUnroll = 8;
// pull ring of the GEMM CTAs (see pull_ring_role)
constexpr int kRingMaxSlots = 8;
constexpr int kRingChunkElems = 4096;                      // default chunk: 8 KB of bf16
constexpr int kRingBytes = 32768;                          // slots = kRingBytes / chunk bytes
constexpr int kRingBarIndex = 24;                          // ring barriers: bars[24..31]
constexpr int kMaxPanels = 1024;

// Device scratch of the fused kernel: zero between launches (the last CTA to leave resets it).
struct Scratch {
  unsigned int panel_done[kMaxPanels];  // copy CTAs that finished panel p
  unsigned int ctas_done;
  int status;  // first error of the last launch that failed (sticky until read)
};

struct Args {
  long long M, N, K;
  __nv_bfloat16* c;
  Scratch* scratch;
  unsigned long long timeout_ns;
  // fused pull
  int fused, num_copy_ctas;
  int inline_copy;          // ring mode: one thread of every GEMM CTA pulls W (no copy CTAs)
  int ring_chunk;           // elements per chunk of the pull ring: 2048, 4096 or 8192
  int ring_mode;            // 0: two warps per CTA, load/store path; 1: one thread, bulk loads
  unsigned int panel_want;  // arrivals that complete a panel
  void* base[PSDEV_MAX_RANKS];
  int rank, world;
  unsigned long long weight_off;  // heap offset of the table's weight buffer
  long long w_elem_off;           // first element of W inside the table
  long long blk;
  int tile_group;  // panels per group of the tile order (1 = panel-major)
};

// Tile order.  Panel-major order (tn = t / tiles_m) makes every CTA of a round read the same
// panel of W at the same time, which lands on a few L2 slices.  With group > 1 the tiles are
// taken in groups of `group` panels with the panel index running fastest, so that a round
// spreads over `group` panels of W and about (CTAs / group) blocks of X.
__device__ __forceinline__ void tile_order(long long t, long long tiles_m, long long tiles_n,
                                           long long group, int* tn, int* tm) {
  const long long per_group = tiles_m * group;
  const long long g = t / per_group, r = t % per_group;
  const long long width = (g + 1) * group <= tiles_n ? group : tiles_n - g * group;
  *tn = (int)(g * group + r % width);
  *tm = (int)(r / width);
}

template <int BN>
struct Cfg {
  static constexpr int kABytes = BM * BK * 2;
  static constexpr int kBBytes = BN * BK * 2;
  static constexpr int kStageBytes = kABytes + kBBytes;
  static constexpr int kStages = BN == 256 ? 4 : 6;
  static constexpr int kTmemCols = 2 * BN;
  static constexpr int kSmemBytes =
      kStages * kStageBytes + 1024 /*align*/ + 256 /*barriers*/ + kRingBytes;
};

__device__ __forceinline__ void report(Scratch* s, int code) { atomicMin(&s->status, code); }

// ---- copy CTA: all-gather of W, panel by panel ----------------------------------------------
template <int BN>
__device__ void copy_role(const Args& a, int copy_idx) {
  const long long panel_elems = (long long)BN * a.K;
  const long long total = a.N * a.K;
  const int npanels = (int)((a.N + BN - 1) / BN);
  char* mine = reinterpret_cast<char*>(a.base[a.rank]) + a.weight_off;
  for (int p = 0; p < npanels; ++p) {
    const long long lo = (long long)p * panel_elems;
    long long hi = lo + panel_elems;
    if (hi > total) hi = total;
    // 16-byte vectors of this panel, interleaved over the copy CTAs
    const long long nvec = (hi - lo) / 8;
    const long long stride = (long long)a.num_copy_ctas * blockDim.x;
    for (long long v0 = (long long)copy_idx * blockDim.x + threadIdx.x; v0 < nvec;
         v0 += stride * kCopyUnroll) {
      uint4 buf[kCopyUnroll];
      long long eoff[kCopyUnroll];
#pragma unroll
      for (int u = 0; u < kCopyUnroll; ++u) {
        const long long v = v0 + u * stride;
        eoff[u] = -1;
        if (v < nvec) {
          const long long e = a.w_elem_off + lo + v * 8;  // element index inside the table
          const int owner = (int)((e / a.blk) % a.world);
          if (owner != a.rank) {
            eoff[u] = e * 2;
            buf[u] = ld_sys_v4(reinterpret_cast<const char*>(a.base[owner]) + a.weight_off + e * 2);
          }
        }
      }
#pragma unroll
      for (int u = 0; u < kCopyUnroll; ++u)
        if (eoff[u] >= 0) st_v4(mine + eoff[u], buf[u]);
    }
    __syncthreads();
    if (threadIdx.x == 0) {
      // the panel is read next by TMA (async proxy) from other CTAs
      fence_proxy_async_global();
      __threadfence();
      atomicAdd(&a.scratch->panel_done[p], 1u);
    }
  }
}

// ---- pull ring: the all-gather of W done by one thread of every GEMM CTA ---------------------
// With no CTA set aside for copying, every SM multiplies.  The blocks of W that other ranks
// own are cut into chunks of at most 8 KB; chunk i belongs to CTA i mod (number of CTAs).  One
// thread per CTA moves its chunks through a ring of buffers (32 KB) in shared memory: an
// untiled bulk load from the owner's memory (over NVLink) into a slot, then a bulk store from
// the slot into this rank's weight buffer.  All slots but one hold loads in flight -- 24 KB,
// about 3.5 MB over 148 SMs, which covers the NVLink round trip -- and the thread itself only
// issues and waits.  Chunks are visited in address order, so once the oldest incomplete chunk
// starts at or beyond the end of panel p this CTA has nothing left in panel p and counts one
// arrival on panel_done[p]; a panel is complete when every CTA has arrived.

// The chunks of the remote blocks of W, in address order.  Elements are indices into the
// table's weight buffer.
struct PullPlan {
  long long e0, e1;   // W = elements [e0, e1)
  long long g0;       // first group of `world` consecutive blocks that touches W
  long long n;        // number of chunk slots (some are empty after clipping to W)
  int blk, cpb, chunk, world, rank;
};
__host__ __device__ inline PullPlan make_pull_plan(long long w_elem_off, long long nk, int blk,
                                                   int world, int rank,
                                                   int chunk_elems = kRingChunkElems) {
  PullPlan pl;
  pl.e0 = w_elem_off;
  pl.e1 = w_elem_off + nk;
  pl.blk = blk;
  pl.world = world;
  pl.rank = rank;
  pl.chunk = blk < chunk_elems ? blk : chunk_elems;
  pl.cpb = (blk + pl.chunk - 1) / pl.chunk;
  pl.g0 = (pl.e0 / blk) / world;
  const long long g1 = ((pl.e1 - 1) / blk) / world;
  pl.n = nk > 0 ? (g1 - pl.g0 + 1) * (world - 1) * pl.cpb : 0;
  return pl;
}
// Chunk slot i -> owner and element range [s, e) (empty when s >= e).  Slot numbers fit in 32
// bits (the launcher checks), which keeps the divisions cheap on the device.
__host__ __device__ inline void pull_chunk(const PullPlan& pl, long long i, int* owner,
                                           long long* s, long long* e) {
  const unsigned int iu = (unsigned int)i;
  const unsigned int q = iu / (unsigned int)pl.cpb;
  const int c = (int)(iu - q * (unsigned int)pl.cpb);
  const unsigned int g = q / (unsigned int)(pl.world - 1);
  const int r = (int)(q - g * (unsigned int)(pl.world - 1));
  const int o = r + (r >= pl.rank ? 1 : 0);
  const long long block = (pl.g0 + g) * pl.world + o;
  long long cs = block * pl.blk + (long long)c * pl.chunk;
  long long ce = cs + pl.chunk;
  const long long be = (block + 1) * pl.blk;
  if (ce > be) ce = be;
  if (cs < pl.e0) cs = pl.e0;
  if (ce > pl.e1) ce = pl.e1;
  *owner = o;
  *s = cs;
  *e = ce;
}

struct ChunkIter {
  long long i, s, e;
  int owner;
  bool valid;
};
__device__ __forceinline__ void chunk_seek(const PullPlan& pl, ChunkIter& it, int stride) {
  // moves to the first non-empty chunk at or after it.i (in steps of `stride`)
  for (; it.i < pl.n; it.i += stride) {
    pull_chunk(pl, it.i, &it.owner, &it.s, &it.e);
    if (it.s < it.e) {
      it.valid = true;
      return;
    }
  }
  it.valid = false;
  it.s = it.e = 0x7fffffffffffffffLL;
}

// Arrivals of one copying agent on the panels of W.  An arrival costs two fences, and every
// agent arrives on every panel, so after the first panels (which the first wave of tiles is
// waiting for) arrivals are made in batches: one pair of fences, then one add per panel.
struct PanelArrivals {
  Scratch* sc;
  long long e0, panel_elems, total;
  int npanels, batch, sig;
  __device__ void init(const Args& a, int bnp) {
    sc = a.scratch;
    e0 = a.w_elem_off;
    panel_elems = (long long)bnp * a.K;
    total = a.N * a.K;
    npanels = (int)((a.N + bnp - 1) / bnp);
    batch = npanels / 16 > 1 ? npanels / 16 : 1;
    sig = 0;
  }
  // Panels that end at or before element `oldest` (the start of the oldest chunk of this agent
  // that may be incomplete) hold nothing more of this agent.
  __device__ int ready(long long oldest) const {
    if (oldest >= e0 + total) return npanels;
    const long long r = (oldest - e0) / panel_elems;
    return r < 0 ? 0 : (int)r;
  }
  __device__ bool due(int rdy) const { return rdy - sig >= (sig < 8 ? 1 : batch); }
  // The caller has made sure that this agent's stores to panels [sig, rdy) are complete.
  __device__ void arrive(int rdy) {
    fence_proxy_async_global();  // the bulk stores went through the async proxy
    __threadfence();
    for (; sig < rdy; ++sig) atomicAdd(&sc->panel_done[sig], 1u);
  }
};

// Executed by TWO threads (of different warps) of CTA `me` of `nctas`: part 0 issues the bulk
// loads, part 1 the bulk stores and the arrivals.  The split keeps the fences of an arrival
// away from the thread that has remote loads in flight.  `ring` is kRingBytes of shared
// memory (16-byte aligned); bar[0..3] count the bytes that land in a slot, bar[4..7] tell the
// loader that a slot has been stored (all initialised with count 1).  BNP: rows of W per panel.
__device__ void pull_ring_role(const Args& a, int part, int me, int nctas, int bnp,
                               unsigned char* ring, uint64_t* bar, volatile int* abort_flag) {
  const PullPlan pl =
      make_pull_plan(a.w_elem_off, a.N * a.K, (int)a.blk, a.world, a.rank, a.ring_chunk);
  const int slot_bytes = a.ring_chunk * 2;
  const int slots = kRingBytes / slot_bytes;  // 2 or 4
  uint64_t* full = bar;
  uint64_t* empty = bar + 4;
  ChunkIter it{me, 0, 0, 0, false};
  chunk_seek(pl, it, nctas);
  long long t = 0;
  if (part == 0) {
    // ---- loader ----
    bool ok = true;
    for (; it.valid; ++t) {
      const int slot = (int)(t % slots);
      const long long round = t / slots;
      if (round > 0 &&
          !mbar_wait_bounded(&empty[slot], (uint32_t)((round - 1) & 1), abort_flag, a.timeout_ns)) {
        ok = false;
        break;
      }
      const uint32_t bytes = (uint32_t)((it.e - it.s) * 2);
      mbar_arrive_expect_tx(&full[slot], bytes);
      bulk_load(ring + slot * slot_bytes,
                reinterpret_cast<const char*>(a.base[it.owner]) + a.weight_off + it.s * 2, bytes,
                &full[slot]);
      it.i += nctas;
      chunk_seek(pl, it, nctas);
    }
    if (!ok || *abort_flag) {
      // loads still in flight must land before the CTA gives up its shared memory
      const unsigned long long t0 = gtimer_ns();
      for (long long u = t > slots ? t - slots : 0; u < t; ++u) {
        const int slot = (int)(u % slots);
        while (!mbar_try_wait(&full[slot], (uint32_t)((u / slots) & 1)) &&
               gtimer_ns() - t0 < a.timeout_ns) {
        }
      }
    }
    return;
  }
  // ---- storer ----
  char* mine = reinterpret_cast<char*>(a.base[a.rank]) + a.weight_off;
  // Stores complete a while after they were issued, so arrivals lag: after the store of chunk
  // k has been committed, only the stores up to chunk k - kSignalLag are awaited, and panels
  // are judged against the start of the oldest chunk that may still be incomplete.
  constexpr int kSignalLag = 3;
  long long lag_s[kSignalLag];  // starts of the last kSignalLag chunks stored, oldest first
#pragma unroll
  for (int i = 0; i < kSignalLag; ++i) lag_s[i] = -1;
  PanelArrivals arr;
  arr.init(a, bnp);
  bool ok = true;
  for (; it.valid; ++t) {
    const int slot = (int)(t % slots);
    if (!mbar_wait_bounded(&full[slot], (uint32_t)((t / slots) & 1), abort_flag, a.timeout_ns)) {
      ok = false;
      break;
    }
    fence_proxy_async_smem();
    bulk_store(mine + it.s * 2, ring + slot * slot_bytes, (uint32_t)((it.e - it.s) * 2));
    bulk_commit();
    // Hand the slot back as soon as the store has read it (a local copy out of shared memory,
    // a fraction of a microsecond): peer reads need every slot in flight to cover their latency.
    bulk_wait_read<0>();
    mbar_arrive(&empty[slot]);
    const long long oldest = lag_s[1] >= 0 ? lag_s[1] : (lag_s[2] >= 0 ? lag_s[2] : it.s);
#pragma unroll
    for (int i = 0; i + 1 < kSignalLag; ++i) lag_s[i] = lag_s[i + 1];
    lag_s[kSignalLag - 1] = it.s;
    const int rdy = arr.ready(oldest);
    if (arr.due(rdy)) {
      bulk_wait<kSignalLag>();  // stores before `oldest` (all but the last kSignalLag) are complete
      arr.arrive(rdy);
    }
    it.i += nctas;
    chunk_seek(pl, it, nctas);
  }
  bulk_wait<0>();
  if (ok) {
    arr.arrive(arr.npanels);
  } else {
    report(a.scratch, PSDEV_ERR_TIMEOUT_PIPE);
  }
}

// The same pull done by whole warps through the load/store path: the lanes of a warp fetch a
// chunk with 16-byte asynchronous copies (global -> shared, several chunks in flight per warp),
// and lane 0 sends each landed chunk on to this rank's weight buffer with one bulk store.
// `ring` is this warp's share of the ring (`ring_bytes`, 2, 4 or 8 chunks).  Arrivals are
// counted per warp.
__device__ __forceinline__ void cp_async_wait_upto(int n) {
  switch (n) {
    case 0: cp_async_wait<0>(); break;
    case 2: cp_async_wait<2>(); break;
    default: cp_async_wait<6>(); break;
  }
}
__device__ void pull_warp_role(const Args& a, int wid, int nwarps, int bnp, unsigned char* ring,
                               int ring_bytes, int lane) {
  const PullPlan pl =
      make_pull_plan(a.w_elem_off, a.N * a.K, (int)a.blk, a.world, a.rank, a.ring_chunk);
  const int slot_bytes = a.ring_chunk * 2;
  const int slots = ring_bytes / slot_bytes;  // 2, 4 or 8
  char* mine = reinterpret_cast<char*>(a.base[a.rank]) + a.weight_off;
  ChunkIter ld{wid, 0, 0, 0, false}, st{wid, 0, 0, 0, false};
  chunk_seek(pl, ld, nwarps);
  st = ld;
  long long nl = 0, ns = 0;
  auto issue = [&](const ChunkIter& c, long long t) {
    const uint32_t bytes = (uint32_t)((c.e - c.s) * 2);
    const char* src = reinterpret_cast<const char*>(a.base[c.owner]) + a.weight_off + c.s * 2;
    unsigned char* dst = ring + (int)(t % slots) * slot_bytes;
    for (uint32_t off = (uint32_t)lane * 16; off < bytes; off += 512)
      cp_async_16(dst + off, src + off);
  };
  // exactly slots-1 groups are committed ahead, empty ones included, so that "all but the
  // newest slots-2 groups" always means "the chunk that is stored next"
  for (int j = 0; j < slots - 1; ++j) {
    if (ld.valid) {
      issue(ld, nl++);
      ld.i += nwarps;
      chunk_seek(pl, ld, nwarps);
    }
    cp_async_commit();
  }
  constexpr int kSignalLag = 3;
  long long lag_s[kSignalLag];
#pragma unroll
  for (int i = 0; i < kSignalLag; ++i) lag_s[i] = -1;
  PanelArrivals arr;
  arr.init(a, bnp);
  while (st.valid) {
    cp_async_wait_upto(slots - 2);  // this lane's pieces of the oldest chunk have landed
    fence_proxy_async_smem();       // ... and may be read by the bulk store
    __syncwarp();
    if (lane == 0) {
      bulk_store(mine + st.s * 2, ring + (int)(ns % slots) * slot_bytes,
                 (uint32_t)((st.e - st.s) * 2));
      bulk_commit();
      const long long oldest = lag_s[1] >= 0 ? lag_s[1] : (lag_s[2] >= 0 ? lag_s[2] : st.s);
#pragma unroll
      for (int i = 0; i + 1 < kSignalLag; ++i) lag_s[i] = lag_s[i + 1];
      lag_s[kSignalLag - 1] = st.s;
      const int rdy = arr.ready(oldest);
      if (arr.due(rdy)) {
        bulk_wait<kSignalLag>();
        arr.arrive(rdy);
      }
      bulk_wait_read<1>();  // the previous store has left its slot: the slot may be refilled
    }
    __syncwarp();
    ++ns;
    st.i += nwarps;
    chunk_seek(pl, st, nwarps);
    if (ld.valid) {
      issue(ld, nl++);
      ld.i += nwarps;
      chunk_seek(pl, ld, nwarps);
    }
    cp_async_commit();
  }
  cp_async_wait<0>();
  if (lane == 0) {
    bulk_wait<0>();
    arr.arrive(arr.npanels);
  }
  __syncwarp();
}

__device__ __forceinline__ bool wait_panel(const Args& a, int p, volatile int* abort_flag) {
  const unsigned int want = a.panel_want;
  const unsigned long long t0 = gtimer_ns();
  while (ld_acquire_gpu_u32(&a.scratch->panel_done[p]) < want) {
    if (*abort_flag) return false;
    if (gtimer_ns() - t0 > a.timeout_ns) {
      *abort_flag = 1;
      return false;
    }
    __nanosleep(64);
  }
  fence_proxy_async_global();
  return true;
}

// ---- GEMM CTA ----------------------------------------------------------------------------------
template <int BN>
__device__ void gemm_role(const Args& a, const CUtensorMap* tmap_x, const CUtensorMap* tmap_w,
                          int gemm_idx, int num_gemm_ctas, unsigned char* smem_raw,
                          volatile int* abort_flag) {
  using C = Cfg<BN>;
  unsigned char* smem = reinterpret_cast<unsigned char*>(
      (reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + C::kStages * C::kStageBytes);
  uint64_t* full_bar = bars;                     // [kStages]
  uint64_t* empty_bar = bars + C::kStages;       // [kStages]
  uint64_t* tmem_full = bars + 2 * C::kStages;   // [2]
  uint64_t* tmem_empty = tmem_full + 2;          // [2]
  uint32_t* tmem_base_slot = reinterpret_cast<uint32_t*>(tmem_empty + 2);
  uint64_t* ring_bar = bars + kRingBarIndex;     // [kRingMaxSlots]
  unsigned char* ring = smem + C::kStages * C::kStageBytes + 256;

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const long long tiles_m = (a.M + BM - 1) / BM;
  const long long tiles_n = (a.N + BN - 1) / BN;
  const long long num_tiles = tiles_m * tiles_n;
  const int num_kb = (int)((a.K + BK - 1) / BK);

  if (threadIdx.x == 0) {
    for (int s = 0; s < C::kStages; ++s) {
      mbar_init(&full_bar[s], 1);
      mbar_init(&empty_bar[s], 1);
    }
    for (int i = 0; i < 2; ++i) {
      mbar_init(&tmem_full[i], 1);
      mbar_init(&tmem_empty[i], 128);
    }
    for (int i = 0; i < kRingMaxSlots; ++i) mbar_init(&ring_bar[i], 1);
    fence_barrier_init();
    prefetch_tmap(tmap_x);
    prefetch_tmap(tmap_w);
  }
  if (warp == 1) {
    tmem_alloc(tmem_base_slot, C::kTmemCols);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_base_slot;

  if (warp == 0) {
    // ================= TMA producer =================
    if (lane == 0) {
      int stage = 0;
      uint32_t phase = 0;
      int armed = 0;  // stages armed in total (for the drain after an abort)
      int last_panel = -1;
      bool ok = true;
      for (long long t = gemm_idx; t < num_tiles && ok; t += num_gemm_ctas) {
        int tn, tm;
        tile_order(t, tiles_m, tiles_n, a.tile_group > 1 ? a.tile_group : 1, &tn, &tm);
        if (a.fused && tn != last_panel) {
          ok = wait_panel(a, tn, abort_flag);
          if (!ok) break;
          last_panel = tn;
        }
        for (int kb = 0; kb < num_kb; ++kb) {
          if (!mbar_wait_bounded(&empty_bar[stage], phase ^ 1, abort_flag, a.timeout_ns)) {
            ok = false;
            break;
          }
          unsigned char* sa = smem + stage * C::kStageBytes;
          unsigned char* sb = sa + C::kABytes;
          mbar_arrive_expect_tx(&full_bar[stage], C::kStageBytes);
          tma_load_2d(sa, tmap_x, kb * BK, tm * BM, &full_bar[stage]);
          tma_load_2d(sb, tmap_w, kb * BK, tn * BN, &full_bar[stage]);
          ++armed;
          if (++stage == C::kStages) { stage = 0; phase ^= 1; }
        }
      }
      if (!ok) {
        report(a.scratch, PSDEV_ERR_TIMEOUT_PIPE);
        // let the copies that are still in flight land before shared memory is released:
        // the last min(armed, kStages) stages may still be receiving bytes
        const int back = armed < C::kStages ? armed : C::kStages;
        int s = stage;
        uint32_t ph = phase;
        for (int i = 0; i < back; ++i) {
          if (--s < 0) { s = C::kStages - 1; ph ^= 1; }
          const unsigned long long t0 = gtimer_ns();
          while (!mbar_try_wait(&full_bar[s], ph) && gtimer_ns() - t0 < 2000000ull) {}
        }
      }
    }
    __syncwarp();
  } else if (warp == 1) {
    // ================= MMA issuer =================
    if (lane == 0) {
      constexpr uint32_t idesc = make_idesc_bf16(BM, BN);
      int stage = 0;
      uint32_t phase = 0;
      long long local = 0;
      bool ok = true;
      for (long long t = gemm_idx; t < num_tiles && ok; t += num_gemm_ctas, ++local) {
        const int acc = (int)(local & 1);
        const uint32_t acc_phase = (uint32_t)((local >> 1) & 1);
        if (!mbar_wait_bounded(&tmem_empty[acc], acc_phase ^ 1, abort_flag, a.timeout_ns)) {
          ok = false;
          break;
        }
        tc_fence_after();
        const uint32_t d_tmem = tmem_base + (uint32_t)(acc * BN);
        for (int kb = 0; kb < num_kb; ++kb) {
          if (!mbar_wait_bounded(&full_bar[stage], phase, abort_flag, a.timeout_ns)) {
            ok = false;
            break;
          }
          tc_fence_after();
          unsigned char* sa = smem + stage * C::kStageBytes;
          const uint64_t da = make_desc_k128(sa);
          const uint64_t db = make_desc_k128(sa + C::kABytes);
#pragma unroll
          for (int k = 0; k < BK / UMMA_K; ++k) {
            // +2 in the address field = 32 bytes = 16 bf16 along K inside the swizzled row
            umma_f16(d_tmem, da + (uint64_t)(2 * k), db + (uint64_t)(2 * k), idesc,
                     (kb | k) != 0 ? 1u : 0u);
          }
          umma_commit(&empty_bar[stage]);  // the stage is free once these MMAs have read it
          if (++stage == C::kStages) { stage = 0; phase ^= 1; }
        }
        if (ok) umma_commit(&tmem_full[acc]);
      }
      if (!ok) report(a.scratch, PSDEV_ERR_TIMEOUT_PIPE);
    }
    __syncwarp();
  } else if (warp < 6) {
    // ================= epilogue (warps 2..5) =================
    const int q = warp & 3;  // tensor-memory lane quarter this warp may read
    long long local = 0;
    bool ok = true;
    for (long long t = gemm_idx; t < num_tiles && ok; t += num_gemm_ctas, ++local) {
      int tn, tm;
        tile_order(t, tiles_m, tiles_n, a.tile_group > 1 ? a.tile_group : 1, &tn, &tm);
      const int acc = (int)(local & 1);
      const uint32_t acc_phase = (uint32_t)((local >> 1) & 1);
      if (!mbar_wait_bounded(&tmem_full[acc], acc_phase, abort_flag, a.timeout_ns)) {
        ok = false;
        break;
      }
      tc_fence_after();
      const long long row = (long long)tm * BM + q * 32 + lane;
      const uint32_t taddr = tmem_base + ((uint32_t)(q * 32) << 16) + (uint32_t)(acc * BN);
#pragma unroll 1
      for (int c0 = 0; c0 < BN; c0 += 32) {
        uint32_t r[32];
        tmem_ld_32x32(taddr + (uint32_t)c0, r);
        tmem_ld_wait();
        const long long col = (long long)tn * BN + c0;
        if (row < a.M) {
          __nv_bfloat16* dst = a.c + row * a.N + col;
#pragma unroll
          for (int j = 0; j < 4; ++j) {
            if (col + j * 8 + 8 <= a.N) {
              uint4 u;
              u.x = f2_to_bf16x2(__uint_as_float(r[8 * j + 0]), __uint_as_float(r[8 * j + 1]));
              u.y = f2_to_bf16x2(__uint_as_float(r[8 * j + 2]), __uint_as_float(r[8 * j + 3]));
              u.z = f2_to_bf16x2(__uint_as_float(r[8 * j + 4]), __uint_as_float(r[8 * j + 5]));
              u.w = f2_to_bf16x2(__uint_as_float(r[8 * j + 6]), __uint_as_float(r[8 * j + 7]));
              *reinterpret_cast<uint4*>(dst + j * 8) = u;
            }
          }
        }
      }
      tc_fence_before();
      mbar_arrive(&tmem_empty[acc]);
    }
    if (!ok && lane == 0) report(a.scratch, PSDEV_ERR_TIMEOUT_PIPE);
  } else if (a.fused && a.inline_copy) {
    // warps 6 and 7: pull W while the other warps multiply
    if (a.ring_mode == 0)
      pull_warp_role(a, gemm_idx * 2 + (warp - 6), num_gemm_ctas * 2, BN,
                     ring + (warp - 6) * (kRingBytes / 2), kRingBytes / 2, lane);
    else if (lane == 0)
      pull_ring_role(a, warp - 6, gemm_idx, num_gemm_ctas, BN, ring, ring_bar, abort_flag);
  }

  // teardown: everyone is done with tensor memory
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  if (warp == 1) tmem_dealloc(tmem_base, C::kTmemCols);
}

// ---- GEMM CTA, 256 x 256 output tile ------------------------------------------------------------
// Same roles as gemm_role, but the CTA owns a 256 x 256 tile: per k-block it loads 256 rows of
// X and 256 rows of W (64 KB) and issues two M=128 MMAs per K step, one per half of the rows,
// into two 256-column accumulators that fill all 512 tensor-memory columns.  An SM can read
// 64 bytes per clock from L2; a 128 x 256 tile needs 96 bytes per tensor-pipe clock and is
// therefore capped near two thirds of the tensor peak, while this shape needs exactly 64.
// The price is that the accumulators are not double buffered: the epilogue of a tile is only
// overlapped with the next tile's first k-blocks half by half, so eight warps drain it.
constexpr int kThreads256 = 384;  // warp 0 TMA, warp 1 MMA, warps 2..9 epilogue, 10..11 pull ring

struct Cfg256 {
  static constexpr int BN = 256, BM2 = 256;
  static constexpr int kABytes = BM2 * BK * 2;   // 32 KB
  static constexpr int kBBytes = BN * BK * 2;    // 32 KB
  static constexpr int kStageBytes = kABytes + kBBytes;
  static constexpr int kStages = 3;
  static constexpr int kTmemCols = 512;
  static constexpr int kSmemBytes = kStages * kStageBytes + 1024 + 256 + kRingBytes;
};

__device__ void gemm_role_256(const Args& a, const CUtensorMap* tmap_x, const CUtensorMap* tmap_w,
                              int gemm_idx, int num_gemm_ctas, unsigned char* smem_raw,
                              volatile int* abort_flag) {
  using C = Cfg256;
  constexpr int BN = C::BN, BM2 = C::BM2;
  unsigned char* smem = reinterpret_cast<unsigned char*>(
      (reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + C::kStages * C::kStageBytes);
  uint64_t* full_bar = bars;                    // [kStages]
  uint64_t* empty_bar = bars + C::kStages;      // [kStages]
  uint64_t* tmem_full = bars + 2 * C::kStages;  // [1]: both halves of the tile are complete
  uint64_t* tmem_empty = tmem_full + 1;         // [2]: half h has been drained
  uint32_t* tmem_base_slot = reinterpret_cast<uint32_t*>(tmem_empty + 2);
  uint64_t* ring_bar = bars + kRingBarIndex;     // [kRingMaxSlots]
  unsigned char* ring = smem + C::kStages * C::kStageBytes + 256;

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const long long tiles_m = (a.M + BM2 - 1) / BM2;
  const long long tiles_n = (a.N + BN - 1) / BN;
  const long long num_tiles = tiles_m * tiles_n;
  const int num_kb = (int)((a.K + BK - 1) / BK);

  if (threadIdx.x == 0) {
    for (int s = 0; s < C::kStages; ++s) {
      mbar_init(&full_bar[s], 1);
      mbar_init(&empty_bar[s], 1);
    }
    mbar_init(&tmem_full[0], 1);
    mbar_init(&tmem_empty[0], 256);  // all eight epilogue warps arrive once per half
    mbar_init(&tmem_empty[1], 256);
    for (int i = 0; i < kRingMaxSlots; ++i) mbar_init(&ring_bar[i], 1);
    fence_barrier_init();
    prefetch_tmap(tmap_x);
    prefetch_tmap(tmap_w);
  }
  if (warp == 1) {
    tmem_alloc(tmem_base_slot, C::kTmemCols);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_base_slot;

  if (warp == 0) {
    if (lane == 0) {
      int stage = 0;
      uint32_t phase = 0;
      int armed = 0, last_panel = -1;
      bool ok = true;
      for (long long t = gemm_idx; t < num_tiles && ok; t += num_gemm_ctas) {
        int tn, tm;
        tile_order(t, tiles_m, tiles_n, a.tile_group > 1 ? a.tile_group : 1, &tn, &tm);
        if (a.fused && tn != last_panel) {
          ok = wait_panel(a, tn, abort_flag);
          if (!ok) break;
          last_panel = tn;
        }
        for (int kb = 0; kb < num_kb; ++kb) {
          if (!mbar_wait_bounded(&empty_bar[stage], phase ^ 1, abort_flag, a.timeout_ns)) {
            ok = false;
            break;
          }
          unsigned char* sa = smem + stage * C::kStageBytes;
          mbar_arrive_expect_tx(&full_bar[stage], C::kStageBytes);
          tma_load_2d(sa, tmap_x, kb * BK, tm * BM2, &full_bar[stage]);
          tma_load_2d(sa + C::kABytes, tmap_w, kb * BK, tn * BN, &full_bar[stage]);
          ++armed;
          if (++stage == C::kStages) { stage = 0; phase ^= 1; }
        }
      }
      if (!ok) {
        report(a.scratch, PSDEV_ERR_TIMEOUT_PIPE);
        const int back = armed < C::kStages ? armed : C::kStages;
        int s = stage;
        uint32_t ph = phase;
        for (int i = 0; i < back; ++i) {
          if (--s < 0) { s = C::kStages - 1; ph ^= 1; }
          const unsigned long long t0 = gtimer_ns();
          while (!mbar_try_wait(&full_bar[s], ph) && gtimer_ns() - t0 < 2000000ull) {}
        }
      }
    }
    __syncwarp();
  } else if (warp == 1) {
    if (lane == 0) {
      constexpr uint32_t idesc = make_idesc_bf16(128, BN);
      int stage = 0;
      uint32_t phase = 0;
      long long local = 0;
      bool ok = true;
      for (long long t = gemm_idx; t < num_tiles && ok; t += num_gemm_ctas, ++local) {
        const uint32_t drained = (uint32_t)(local & 1) ^ 1;  // parity of the previous drain
        if (!mbar_wait_bounded(&tmem_empty[0], drained, abort_flag, a.timeout_ns)) {
          ok = false;
          break;
        }
        bool half1_free = false;
        for (int kb = 0; kb < num_kb; ++kb) {
          if (!mbar_wait_bounded(&full_bar[stage], phase, abort_flag, a.timeout_ns)) {
            ok = false;
            break;
          }
          tc_fence_after();
          unsigned char* sa = smem + stage * C::kStageBytes;
          const uint64_t da0 = make_desc_k128(sa);
          const uint64_t da1 = make_desc_k128(sa + 128 * BK * 2);
          const uint64_t db = make_desc_k128(sa + C::kABytes);
#pragma unroll
          for (int k = 0; k < BK / UMMA_K; ++k)
            umma_f16(tmem_base, da0 + (uint64_t)(2 * k), db + (uint64_t)(2 * k), idesc,
                     (kb | k) != 0 ? 1u : 0u);
          if (!half1_free) {
            // the second half may still be draining from the previous tile
            if (!mbar_wait_bounded(&tmem_empty[1], drained, abort_flag, a.timeout_ns)) {
              ok = false;
              break;
            }
            tc_fence_after();
            half1_free = true;
          }
#pragma unroll
          for (int k = 0; k < BK / UMMA_K; ++k)
            umma_f16(tmem_base + (uint32_t)BN, da1 + (uint64_t)(2 * k), db + (uint64_t)(2 * k),
                     idesc, (kb | k) != 0 ? 1u : 0u);
          umma_commit(&empty_bar[stage]);
          if (++stage == C::kStages) { stage = 0; phase ^= 1; }
        }
        if (ok) umma_commit(&tmem_full[0]);
      }
      if (!ok) report(a.scratch, PSDEV_ERR_TIMEOUT_PIPE);
    }
    __syncwarp();
  } else if (warp < 10) {
    // epilogue: warp w reads lane quarter (w & 3); warps 2..5 take columns [0,128) of each
    // half, warps 6..9 columns [128,256)
    const int q = warp & 3;
    const int col_half = (warp - 2) >> 2;
    long long local = 0;
    bool ok = true;
    for (long long t = gemm_idx; t < num_tiles && ok; t += num_gemm_ctas, ++local) {
      int tn, tm;
        tile_order(t, tiles_m, tiles_n, a.tile_group > 1 ? a.tile_group : 1, &tn, &tm);
      if (!mbar_wait_bounded(&tmem_full[0], (uint32_t)(local & 1), abort_flag, a.timeout_ns)) {
        ok = false;
        break;
      }
      __syncwarp();
      tc_fence_after();
#pragma unroll 1
      for (int h = 0; h < 2; ++h) {
        const long long row = (long long)tm * BM2 + h * 128 + q * 32 + lane;
        const uint32_t taddr = tmem_base + ((uint32_t)(q * 32) << 16) + (uint32_t)(h * BN);
#pragma unroll 1
        for (int c0 = col_half * 128; c0 < col_half * 128 + 128; c0 += 32) {
          uint32_t r[32];
          tmem_ld_32x32(taddr + (uint32_t)c0, r);
          tmem_ld_wait();
          const long long col = (long long)tn * BN + c0;
          if (row < a.M) {
            __nv_bfloat16* dst = a.c + row * a.N + col;
#pragma unroll
            for (int j = 0; j < 4; ++j) {
              if (col + j * 8 + 8 <= a.N) {
                uint4 u;
                u.x = f2_to_bf16x2(__uint_as_float(r[8 * j + 0]), __uint_as_float(r[8 * j + 1]));
                u.y = f2_to_bf16x2(__uint_as_float(r[8 * j + 2]), __uint_as_float(r[8 * j + 3]));
                u.z = f2_to_bf16x2(__uint_as_float(r[8 * j + 4]), __uint_as_float(r[8 * j + 5]));
                u.w = f2_to_bf16x2(__uint_as_float(r[8 * j + 6]), __uint_as_float(r[8 * j + 7]));
                *reinterpret_cast<uint4*>(dst + j * 8) = u;
              }
            }
          }
        }
        tc_fence_before();
        mbar_arrive(&tmem_empty[h]);  // 256 arrivals (8 warps) free half h for the next tile
      }
    }
    if (!ok && lane == 0) report(a.scratch, PSDEV_ERR_TIMEOUT_PIPE);
  } else if (a.fused && a.inline_copy) {
    // warps 10 and 11: pull W while the other warps multiply
    if (a.ring_mode == 0)
      pull_warp_role(a, gemm_idx * 2 + (warp - 10), num_gemm_ctas * 2, BN,
                     ring + (warp - 10) * (kRingBytes / 2), kRingBytes / 2, lane);
    else if (lane == 0)
      pull_ring_role(a, warp - 10, gemm_idx, num_gemm_ctas, BN, ring, ring_bar, abort_flag);
  }

  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  if (warp == 1) tmem_dealloc(tmem_base, C::kTmemCols);
}

__global__ void __launch_bounds__(kThreads256, 1)
    pull_gemm256_kernel(const __grid_constant__ Args a, const __grid_constant__ CUtensorMap tmap_x,
                        const __grid_constant__ CUtensorMap tmap_w) {
  extern __shared__ unsigned char smem_raw[];
  __shared__ int s_abort;
  __shared__ int s_last;
  if (threadIdx.x == 0) s_abort = 0;
  __syncthreads();
  const int ncopy = a.fused ? a.num_copy_ctas : 0;
  if ((int)blockIdx.x < ncopy) {
    copy_role<256>(a, (int)blockIdx.x);
  } else {
    gemm_role_256(a, &tmap_x, &tmap_w, (int)blockIdx.x - ncopy, (int)gridDim.x - ncopy, smem_raw,
                  &s_abort);
  }
  __syncthreads();
  if (threadIdx.x == 0) {
    __threadfence();
    s_last = (atomicAdd(&a.scratch->ctas_done, 1u) == gridDim.x - 1);
    if (s_last) {
      const int npanels = (int)((a.N + 255) / 256);
      for (int p = 0; p < npanels; ++p) a.scratch->panel_done[p] = 0;
      a.scratch->ctas_done = 0;
      __threadfence();
    }
  }
}

// ---- GEMM on CTA pairs (tcgen05 cta_group::2) -------------------------------------------------
// Two CTAs of a 2-CTA cluster own one 256 x 256 output tile: CTA r of the pair loads rows
// [r*128, r*128+128) of the X tile and of the W tile (32 KB per k-block instead of 48 KB, i.e.
// the 64 bytes per tensor-pipe clock an SM can take from L2), keeps the accumulators of its
// 128 rows in its own tensor memory (two buffers of 256 columns, so the epilogue overlaps the
// next tile), and the even CTA issues one M=256 MMA per K step for both.  Loads carry no
// cluster multicast: each CTA fetches its own halves; only the completion counts and the
// MMA-done signals cross between the two CTAs.
// kRing: room for the pull ring of the fused form; the plain GEMM spends it on a seventh stage.
template <bool kRing>
struct CfgPairT {
  static constexpr int BN = 256;
  static constexpr int kABytes = 128 * BK * 2;  // this CTA's 128 rows of X
  static constexpr int kBBytes = 128 * BK * 2;  // this CTA's 128 rows of W
  static constexpr int kStageBytes = kABytes + kBBytes;
  static constexpr int kStages = kRing ? 6 : 7;
  static constexpr int kTmemCols = 512;
  static constexpr int kSmemBytes =
      kStages * kStageBytes + 1024 + 256 + (kRing ? kRingBytes : 0);
};
using CfgPair = CfgPairT<true>;

template <bool kRing>
__device__ void gemm_role_pair(const Args& a, const CUtensorMap* tmap_x, const CUtensorMap* tmap_w,
                               int pair_idx, int num_pairs, unsigned char* smem_raw,
                               volatile int* abort_flag) {
  using C = CfgPairT<kRing>;
  constexpr int BN = C::BN;
  static_assert(2 * C::kStages + 5 <= kRingBarIndex, "pipeline barriers overlap the ring's");
  unsigned char* smem = reinterpret_cast<unsigned char*>(
      (reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + C::kStages * C::kStageBytes);
  uint64_t* full_bar = bars;                    // [kStages]  used in the leader CTA
  uint64_t* empty_bar = bars + C::kStages;      // [kStages]  one copy per CTA
  uint64_t* tmem_full = bars + 2 * C::kStages;  // [2]        one copy per CTA
  uint64_t* tmem_empty = tmem_full + 2;         // [2]        used in the leader CTA
  uint32_t* tmem_base_slot = reinterpret_cast<uint32_t*>(tmem_empty + 2);
  uint64_t* ring_bar = bars + kRingBarIndex;     // [kRingMaxSlots]
  unsigned char* ring = smem + C::kStages * C::kStageBytes + 256;

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const uint32_t cta = cluster_ctarank();  // 0 = leader
  const long long tiles_m = (a.M + 255) / 256;
  const long long tiles_n = (a.N + BN - 1) / BN;
  const long long num_tiles = tiles_m * tiles_n;
  const int num_kb = (int)((a.K + BK - 1) / BK);
  // Work items.  The tiles of the last, partly filled round are cut along N into 2 or 4 pieces
  // when that lets every piece have a pair of its own: the round then lasts a half or a
  // quarter of a tile time instead of a whole one.  (A piece of n columns needs n/2 rows of W in
  // each CTA: the usual 128-row box is loaded and the MMA reads its first n/2 rows.)
  const long long rest = num_tiles % num_pairs;
  int split = 1;
  if (rest != 0 && num_tiles > num_pairs) {
    if (rest * 4 <= num_pairs) split = 4;
    else if (rest * 2 <= num_pairs) split = 2;
  }
  const long long num_whole = split > 1 ? num_tiles - rest : num_tiles;
  const long long num_items = num_whole + (split > 1 ? rest * split : 0);
  const long long group = a.tile_group > 1 ? a.tile_group : 1;
  auto tile_of = [&](long long t, int* tn, int* tm) {
    tile_order(t, tiles_m, tiles_n, group, tn, tm);
  };
  // item -> (tile, first column inside the tile, columns)
  auto item_of = [&](long long i, long long* t, int* n_off, int* n_len) {
    if (i < num_whole) {
      *t = i;
      *n_off = 0;
      *n_len = BN;
    } else {
      const long long j = i - num_whole;
      *t = num_whole + j / split;
      *n_len = BN / split;
      *n_off = (int)(j % split) * *n_len;
    }
  };

  if (threadIdx.x == 0) {
    for (int s = 0; s < C::kStages; ++s) {
      mbar_init(&full_bar[s], 1);   // the leader's arrive.expect_tx; bytes come from both CTAs
      mbar_init(&empty_bar[s], 1);  // the leader's commit, delivered to both CTAs
    }
    for (int i = 0; i < 2; ++i) {
      mbar_init(&tmem_full[i], 1);
      mbar_init(&tmem_empty[i], 256);  // 128 epilogue threads of each CTA
    }
    for (int i = 0; i < kRingMaxSlots; ++i) mbar_init(&ring_bar[i], 1);
    fence_barrier_init();
    prefetch_tmap(tmap_x);
    prefetch_tmap(tmap_w);
  }
  if (warp == 1) {
    tmem_alloc_pair(tmem_base_slot, C::kTmemCols);
    tmem_relinquish_pair();
  }
  tc_fence_before();
  cluster_sync_all();  // both CTAs' barriers exist before anything can signal them
  tc_fence_after();
  const uint32_t tmem_base = *tmem_base_slot;

  if (warp == 0) {
    // ================= TMA producer (both CTAs) =================
    if (lane == 0) {
      int stage = 0;
      uint32_t phase = 0;
      int last_panel = -1;
      bool ok = true;
      for (long long it = pair_idx; it < num_items && ok; it += num_pairs) {
        long long t;
        int n_off, n_len;
        item_of(it, &t, &n_off, &n_len);
        int tn, tm;
        tile_of(t, &tn, &tm);
        if (a.fused && tn != last_panel) {
          ok = wait_panel(a, tn, abort_flag);
          if (!ok) break;
          last_panel = tn;
        }
        for (int kb = 0; kb < num_kb; ++kb) {
          if (!mbar_wait_bounded(&empty_bar[stage], phase ^ 1, abort_flag, a.timeout_ns)) {
            ok = false;
            break;
          }
          unsigned char* sa = smem + stage * C::kStageBytes;
          if (cta == 0) mbar_arrive_expect_tx(&full_bar[stage], 2 * C::kStageBytes);
          tma_load_2d_pair(sa, tmap_x, kb * BK, tm * 256 + (int)cta * 128, &full_bar[stage]);
          tma_load_2d_pair(sa + C::kABytes, tmap_w, kb * BK,
                           tn * BN + n_off + (int)cta * (n_len / 2), &full_bar[stage]);
          if (++stage == C::kStages) { stage = 0; phase ^= 1; }
        }
      }
      if (!ok) report(a.scratch, PSDEV_ERR_TIMEOUT_PIPE);
    }
    __syncwarp();
  } else if (warp == 1) {
    // ================= MMA issuer (leader CTA only) =================
    if (lane == 0 && cta == 0) {
      int stage = 0;
      uint32_t phase = 0;
      long long local = 0;
      bool ok = true;
      for (long long it = pair_idx; it < num_items && ok; it += num_pairs, ++local) {
        long long t;
        int n_off, n_len;
        item_of(it, &t, &n_off, &n_len);
        const uint32_t idesc = make_idesc_bf16(256, n_len);
        const int acc = (int)(local & 1);
        const uint32_t acc_phase = (uint32_t)((local >> 1) & 1);
        if (!mbar_wait_bounded(&tmem_empty[acc], acc_phase ^ 1, abort_flag, a.timeout_ns)) {
          ok = false;
          break;
        }
        tc_fence_after();
        const uint32_t d_tmem = tmem_base + (uint32_t)(acc * BN);
        for (int kb = 0; kb < num_kb; ++kb) {
          if (!mbar_wait_bounded(&full_bar[stage], phase, abort_flag, a.timeout_ns)) {
            ok = false;
            break;
          }
          tc_fence_after();
          unsigned char* sa = smem + stage * C::kStageBytes;
          const uint64_t da = make_desc_k128(sa);
          const uint64_t db = make_desc_k128(sa + C::kABytes);
#pragma unroll
          for (int k = 0; k < BK / UMMA_K; ++k)
            umma_f16_pair(d_tmem, da + (uint64_t)(2 * k), db + (uint64_t)(2 * k), idesc,
                          (kb | k) != 0 ? 1u : 0u);
          umma_commit_pair(&empty_bar[stage]);  // frees the stage in both CTAs
          if (++stage == C::kStages) { stage = 0; phase ^= 1; }
        }
        if (ok) umma_commit_pair(&tmem_full[acc]);  // wakes the epilogues of both CTAs
      }
      if (!ok) report(a.scratch, PSDEV_ERR_TIMEOUT_PIPE);
    }
    __syncwarp();
  } else if (warp < 6) {
    // ================= epilogue (warps 2..5 of both CTAs) =================
    const int q = warp & 3;
    long long local = 0;
    bool ok = true;
    for (long long it = pair_idx; it < num_items && ok; it += num_pairs, ++local) {
      long long t;
      int n_off, n_len;
      item_of(it, &t, &n_off, &n_len);
      int tn, tm;
        tile_of(t, &tn, &tm);
      const int acc = (int)(local & 1);
      const uint32_t acc_phase = (uint32_t)((local >> 1) & 1);
      if (!mbar_wait_bounded(&tmem_full[acc], acc_phase, abort_flag, a.timeout_ns)) {
        ok = false;
        break;
      }
      __syncwarp();
      tc_fence_after();
      const long long row = (long long)tm * 256 + (long long)cta * 128 + q * 32 + lane;
      const uint32_t taddr = tmem_base + ((uint32_t)(q * 32) << 16) + (uint32_t)(acc * BN);
#pragma unroll 1
      for (int c0 = 0; c0 < n_len; c0 += 32) {
        uint32_t r[32];
        tmem_ld_32x32(taddr + (uint32_t)c0, r);
        tmem_ld_wait();
        const long long col = (long long)tn * BN + n_off + c0;
        if (row < a.M) {
          __nv_bfloat16* dst = a.c + row * a.N + col;
#pragma unroll
          for (int j = 0; j < 4; ++j) {
            if (col + j * 8 + 8 <= a.N) {
              uint4 u;
              u.x = f2_to_bf16x2(__uint_as_float(r[8 * j + 0]), __uint_as_float(r[8 * j + 1]));
              u.y = f2_to_bf16x2(__uint_as_float(r[8 * j + 2]), __uint_as_float(r[8 * j + 3]));
              u.z = f2_to_bf16x2(__uint_as_float(r[8 * j + 4]), __uint_as_float(r[8 * j + 5]));
              u.w = f2_to_bf16x2(__uint_as_float(r[8 * j + 6]), __uint_as_float(r[8 * j + 7]));
              *reinterpret_cast<uint4*>(dst + j * 8) = u;
            }
          }
        }
      }
      tc_fence_before();
      mbar_arrive_leader(&tmem_empty[acc]);  // counted on the leader, where the MMAs are issued
    }
    if (!ok && lane == 0) report(a.scratch, PSDEV_ERR_TIMEOUT_PIPE);
  } else if (kRing && a.fused && a.inline_copy) {
    // warps 6 and 7: pull W while the other warps multiply
    const int cta_lin = pair_idx * 2 + (int)cta;
    if (a.ring_mode == 0)
      pull_warp_role(a, cta_lin * 2 + (warp - 6), num_pairs * 4, BN,
                     ring + (warp - 6) * (kRingBytes / 2), kRingBytes / 2, lane);
    else if (lane == 0)
      pull_ring_role(a, warp - 6, cta_lin, num_pairs * 2, BN, ring, ring_bar, abort_flag);
  }

  // teardown: neither CTA may free its tensor memory while the other might still be used by
  // a pair MMA, so the whole cluster meets first
  tc_fence_before();
  cluster_sync_all();
  tc_fence_after();
  if (warp == 1) tmem_dealloc_pair(tmem_base, C::kTmemCols);
}

// Grid: [copy CTAs (even count)][GEMM CTA pairs], clusters of 2 along x.
template <bool kRing>
__global__ void __launch_bounds__(kThreads, 1)
    pull_gemm_pair_kernel(const __grid_constant__ Args a,
                          const __grid_constant__ CUtensorMap tmap_x,
                          const __grid_constant__ CUtensorMap tmap_w) {
  extern __shared__ unsigned char smem_raw[];
  __shared__ int s_abort;
  __shared__ int s_last;
  if (threadIdx.x == 0) s_abort = 0;
  __syncthreads();
  const int ncopy = a.fused ? a.num_copy_ctas : 0;
  if ((int)blockIdx.x < ncopy) {
    copy_role<256>(a, (int)blockIdx.x);
  } else {
    gemm_role_pair<kRing>(a, &tmap_x, &tmap_w, ((int)blockIdx.x - ncopy) >> 1,
                          ((int)gridDim.x - ncopy) >> 1, smem_raw, &s_abort);
  }
  __syncthreads();
  if (threadIdx.x == 0) {
    __threadfence();
    s_last = (atomicAdd(&a.scratch->ctas_done, 1u) == gridDim.x - 1);
    if (s_last) {
      const int npanels = (int)((a.N + 255) / 256);
      for (int p = 0; p < npanels; ++p) a.scratch->panel_done[p] = 0;
      a.scratch->ctas_done = 0;
      __threadfence();
    }
  }
}

// Grid: [num_copy_ctas copy CTAs][GEMM CTAs], 256 threads each.  GEMM CTAs use six warps;
// the last two only take part in the block-wide barriers.
//
// No flag is exchanged between ranks here.  The fused form must follow, on the same stream,
// a push that published the owners' blocks (PSDEV_OP_PUSH | PSDEV_OP_PUBLISH): that kernel
// returns only after every rank has finished publishing, and the entry rendezvous of the
// next push on the channel keeps owners from overwriting a shard that a peer still reads.
template <int BN>
__global__ void __launch_bounds__(kThreads, 1)
    pull_gemm_kernel(const __grid_constant__ Args a, const __grid_constant__ CUtensorMap tmap_x,
                     const __grid_constant__ CUtensorMap tmap_w) {
  extern __shared__ unsigned char smem_raw[];
  __shared__ int s_abort;
  __shared__ int s_last;
  if (threadIdx.x == 0) s_abort = 0;
  __syncthreads();
  const int ncopy = a.fused ? a.num_copy_ctas : 0;
  if ((int)blockIdx.x < ncopy) {
    copy_role<BN>(a, (int)blockIdx.x);
  } else {
    gemm_role<BN>(a, &tmap_x, &tmap_w, (int)blockIdx.x - ncopy, (int)gridDim.x - ncopy,
                  smem_raw, &s_abort);
  }
  // the last CTA to leave puts the scratch back to zero for the next launch
  __syncthreads();
  if (threadIdx.x == 0) {
    __threadfence();
    s_last = (atomicAdd(&a.scratch->ctas_done, 1u) == gridDim.x - 1);
    if (s_last) {
      const int npanels = (int)((a.N + BN - 1) / BN);
      for (int p = 0; p < npanels; ++p) a.scratch->panel_done[p] = 0;
      a.scratch->ctas_done = 0;
      __threadfence();
    }
  }
}

}  // namespace gemm
}  // namespace psdev

// ================================== host side ===================================================
namespace psdev {
namespace gemm {

using EncodeFn = CUresult (*)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*,
                              const cuuint64_t*, const cuuint64_t*, const cuuint32_t*,
                              const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                              CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

static EncodeFn encode_fn() {
  static EncodeFn fn = [] {
    void* p = nullptr;
    cudaDriverEntryPointQueryResult q;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) !=
            cudaSuccess || q != cudaDriverEntryPointSuccess)
      p = nullptr;
    return reinterpret_cast<EncodeFn>(p);
  }();
  return fn;
}

// Row-major [rows, cols] bf16 tensor, tiles of box_rows x 64 columns, 128-byte swizzle,
// out-of-bounds elements read as zero.
static int make_tmap(CUtensorMap* m, const void* ptr, long long rows, long long cols,
                     int box_rows) {
  EncodeFn fn = encode_fn();
  if (!fn) return PSDEV_ERR_UNSUPPORTED;
  cuuint64_t dims[2] = {(cuuint64_t)cols, (cuuint64_t)rows};
  cuuint64_t strides[1] = {(cuuint64_t)cols * 2};
  cuuint32_t box[2] = {(cuuint32_t)BK, (cuuint32_t)box_rows};
  cuuint32_t estr[2] = {1, 1};
  CUresult r = fn(m, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(ptr), dims, strides,
                  box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B,
                  CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  return r == CUDA_SUCCESS ? 0 : PSDEV_ERR_ARG;
}

// One scratch block per device, allocated on first use and kept until the process exits.
static Scratch* scratch_for_current_device(int* err) {
  static std::mutex mu;
  static Scratch* table[64] = {};
  int dev = 0;
  cudaGetDevice(&dev);
  std::lock_guard<std::mutex> lk(mu);
  if (dev < 0 || dev >= 64) { *err = PSDEV_ERR_ARG; return nullptr; }
  if (!table[dev]) {
    Scratch* s = nullptr;
    cudaError_t e = cudaMalloc(&s, sizeof(Scratch));
    if (e == cudaSuccess) e = cudaMemset(s, 0, sizeof(Scratch));
    if (e != cudaSuccess) { *err = (int)e; return nullptr; }
    table[dev] = s;
  }
  return table[dev];
}

// One launch; `cluster` CTAs per cluster along x.  In ring mode every CTA's pull thread feeds
// every other CTA, so the launch asks for all CTAs to be resident together (cooperative).
typedef void (*GemmKernel)(const Args, const CUtensorMap, const CUtensorMap);
static int launch_ex(GemmKernel k, const Args& a, const CUtensorMap& tx, const CUtensorMap& tw,
                     int grid, int threads, int smem, int cluster, cudaStream_t s) {
  cudaLaunchConfig_t cfg{};
  cfg.gridDim = dim3((unsigned)grid, 1, 1);
  cfg.blockDim = dim3((unsigned)threads, 1, 1);
  cfg.dynamicSmemBytes = (size_t)smem;
  cfg.stream = s;
  cudaLaunchAttribute attr[2];
  int n = 0;
  if (cluster > 1) {
    attr[n].id = cudaLaunchAttributeClusterDimension;
    attr[n].val.clusterDim.x = (unsigned)cluster;
    attr[n].val.clusterDim.y = 1;
    attr[n].val.clusterDim.z = 1;
    ++n;
  }
  // PSB200_PULL_GEMM_COOP=0 drops the co-residency request (measurements only: without it
  // a busy GPU can leave a CTA waiting for a pull thread that has not been scheduled)
  static const bool coop = [] {
    const char* e = getenv("PSB200_PULL_GEMM_COOP");
    return !(e && e[0] == '0');
  }();
  if (a.fused && a.inline_copy && coop) {
    attr[n].id = cudaLaunchAttributeCooperative;
    attr[n].val.cooperative = 1;
    ++n;
  }
  cfg.attrs = attr;
  cfg.numAttrs = (unsigned)n;
  cudaError_t e = cudaLaunchKernelEx(&cfg, k, a, tx, tw);
  g_launches.fetch_add(1, std::memory_order_relaxed);
  return (int)e;
}

template <int BN>
static int launch(const Args& a, const CUtensorMap& tx, const CUtensorMap& tw, int grid,
                  cudaStream_t s) {
  // (set once per device; the attribute call is idempotent, the flag is atomic because the
  // entry points may be used from several host threads)
  static std::atomic<bool> attr_set[64];
  int dev = 0;
  cudaGetDevice(&dev);
  if (!attr_set[dev & 63].load(std::memory_order_acquire)) {
    cudaError_t e = cudaFuncSetAttribute(pull_gemm_kernel<BN>,
                                         cudaFuncAttributeMaxDynamicSharedMemorySize,
                                         Cfg<BN>::kSmemBytes);
    if (e != cudaSuccess) return (int)e;
    attr_set[dev & 63].store(true, std::memory_order_release);
  }
  return launch_ex(pull_gemm_kernel<BN>, a, tx, tw, grid, kThreads, Cfg<BN>::kSmemBytes, 1, s);
}

static int launch256(const Args& a, const CUtensorMap& tx, const CUtensorMap& tw, int grid,
                     cudaStream_t s) {
  // (set once per device; the attribute call is idempotent, the flag is atomic because the
  // entry points may be used from several host threads)
  static std::atomic<bool> attr_set[64];
  int dev = 0;
  cudaGetDevice(&dev);
  if (!attr_set[dev & 63].load(std::memory_order_acquire)) {
    cudaError_t e = cudaFuncSetAttribute(pull_gemm256_kernel,
                                         cudaFuncAttributeMaxDynamicSharedMemorySize,
                                         Cfg256::kSmemBytes);
    if (e != cudaSuccess) return (int)e;
    attr_set[dev & 63].store(true, std::memory_order_release);
  }
  return launch_ex(pull_gemm256_kernel, a, tx, tw, grid, kThreads256, Cfg256::kSmemBytes, 1, s);
}

template <bool kRing>
static int launch_pair_t(const Args& a, const CUtensorMap& tx, const CUtensorMap& tw, int grid,
                         cudaStream_t s) {
  static std::atomic<bool> attr_set[64];
  int dev = 0;
  cudaGetDevice(&dev);
  if (!attr_set[dev & 63].load(std::memory_order_acquire)) {
    cudaError_t e = cudaFuncSetAttribute(pull_gemm_pair_kernel<kRing>,
                                         cudaFuncAttributeMaxDynamicSharedMemorySize,
                                         CfgPairT<kRing>::kSmemBytes);
    if (e != cudaSuccess) return (int)e;
    attr_set[dev & 63].store(true, std::memory_order_release);
  }
  return launch_ex(pull_gemm_pair_kernel<kRing>, a, tx, tw, grid, kThreads,
                   CfgPairT<kRing>::kSmemBytes, 2, s);
}
static int launch_pair(const Args& a, const CUtensorMap& tx, const CUtensorMap& tw, int grid,
                       cudaStream_t s) {
  // (the plain GEMM needs no pull ring and could spend its room on a seventh pipeline stage)
  static const int stages_env = [] {
    const char* e = getenv("PSB200_GEMM_PAIR_STAGES");
    return e ? atoi(e) : 0;
  }();
  // measured on 16384x3072x1024: six stages 1258 TFLOP/s, seven (possible without the pull
  // ring) 1228-1243: the seventh stage stays an option (PSB200_GEMM_PAIR_STAGES=7)
  if (a.fused || stages_env != 7) return launch_pair_t<true>(a, tx, tw, grid, s);
  return launch_pair_t<false>(a, tx, tw, grid, s);
}

// Output-tile height used by run(): 128 (double-buffered accumulators) or 256 (twice the
// reuse of W per byte loaded).  0 = choose by shape.
static std::atomic<int> g_tile_m{0};

static int pick_tile_m(long long M, long long N, long long K) {
  int t = g_tile_m.load();
  if (t == 0) {
    const char* e = getenv("PSB200_GEMM_TILE");
    t = e ? atoi(e) : 0;
  }
  if (t == 2) return (N >= 256 && M >= 256) ? 2 : 128;  // 2 = CTA pairs
  if (t == 128 || t == 256) return (t == 256 && N >= 256 && M >= 256) ? 256 : 128;
  // by shape (measured on one B200, bf16, TFLOP/s):
  //   16384x3072x1024: pairs 1198, 128-row tile 1070, 256-row tile 868
  //   16384x4096x1024: pairs 1398, 128-row tile 1169
  //   8192x8192x8192 : 256-row tile 1533, pairs 1477, 128-row tile 1341
  // CTA pairs whenever there is at least one 256 x 256 tile per pair of SMs; the one-CTA
  // 256-row tile for long reductions, where its exposed epilogue is amortised.
  const long long tiles256 = ((M + 255) / 256) * ((N + 255) / 256);
  if (N >= 256 && M >= 256 && K >= 4096 && tiles256 >= 2 * 148) return 256;
  if (N >= 256 && M >= 256 && tiles256 >= 74) return 2;
  return 128;
}

static int run(Args a, const void* x, const void* w, int num_ctas, cudaStream_t s) {
  if (a.M <= 0 || a.N <= 0 || a.K <= 0 || (a.N & 7) || (a.K & 7)) return PSDEV_ERR_ARG;
  if (((uintptr_t)x & 15) || ((uintptr_t)w & 15) || ((uintptr_t)a.c & 15)) return PSDEV_ERR_ARG;
  int err = 0;
  a.scratch = scratch_for_current_device(&err);
  if (!a.scratch) return err;
  const int variant = pick_tile_m(a.M, a.N, a.K);
  const bool pair = (variant == 2);
  const int tile_m = pair ? 256 : variant;  // rows of X per output tile (per pair for pairs)
  const int BN = (tile_m == 256 || a.N % 256 == 0 || a.N > 1024) ? 256 : 128;
  if ((a.N + BN - 1) / BN >= kMaxPanels) return PSDEV_ERR_UNSUPPORTED;
  CUtensorMap tx, tw;
  // a CTA of a pair loads 128 rows of each operand per k-block
  int rc = make_tmap(&tx, x, a.M, a.K, pair ? 128 : tile_m);
  if (rc) return rc;
  rc = make_tmap(&tw, w, a.N, a.K, pair ? 128 : BN);
  if (rc) return rc;
  int sms = 148;
  int dev = 0;
  cudaGetDevice(&dev);
  cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
  const long long tiles = ((a.M + tile_m - 1) / tile_m) * ((a.N + BN - 1) / BN);
  const int avail = num_ctas > 0 ? num_ctas : sms;
  // One launch of the chosen variant with `copy` CTAs set aside (0: ring mode or not fused).
  auto go = [&](int copy) -> int {
    if (pair) {
      // clusters of two: even number of copy CTAs, GEMM CTAs in pairs (one tile per pair)
      copy = (copy + 1) & ~1;
      int pairs = avail / 2 - copy / 2;
      if (pairs < 1) pairs = 1;
      if (tiles < pairs) pairs = (int)tiles;
      a.num_copy_ctas = copy;
      a.panel_want = (unsigned int)(copy ? copy : 2 * pairs * (a.ring_mode == 0 ? 2 : 1));
      return launch_pair(a, tx, tw, 2 * pairs + copy, s);
    }
    int gemm_ctas = avail > copy + 1 ? avail - copy : 1;
    if (tiles < gemm_ctas) gemm_ctas = (int)tiles;
    a.num_copy_ctas = copy;
    a.panel_want = (unsigned int)(copy ? copy : gemm_ctas * (a.ring_mode == 0 ? 2 : 1));
    const int grid = gemm_ctas + copy;
    if (tile_m == 256) return launch256(a, tx, tw, grid, s);
    return BN == 256 ? launch<256>(a, tx, tw, grid, s) : launch<128>(a, tx, tw, grid, s);
  };
  {
    // a GEMM that waits for panels of W to arrive takes them in order; otherwise groups of 8
    static const int group_env = [] {
      const char* e = getenv("PSB200_GEMM_GROUP");
      return e ? atoi(e) : 0;
    }();
    const long long tn_count = (a.N + BN - 1) / BN;
    // measured: with up to 16 panels the best order runs through all of them for each block of
    // X rows (16384x3072x1024: 1213 / 1242 / 1307 / 1325 TFLOP/s for groups of 2 / 4 / 8 / 16);
    // with more, groups of 8 (8192^3: 1591 against 1568 with 16)
    long long group = group_env > 0 ? group_env : (tn_count <= 16 ? tn_count : 8);
    if (group > tn_count) group = tn_count;
    a.tile_group = a.fused ? 1 : (int)group;
  }
  if (!a.fused) {
    a.inline_copy = 0;
    return go(0);
  }
  if (a.inline_copy &&
      make_pull_plan(a.w_elem_off, a.N * a.K, (int)a.blk, a.world, a.rank, a.ring_chunk).n >=
          (1ll << 31)) {
    a.inline_copy = 0;  // chunk slots are numbered in 32 bits on the device
    a.num_copy_ctas = 16;
  }
  if (a.inline_copy) {
    // ring mode: no copy CTAs, one thread of every GEMM CTA pulls W
    if (go(0) == 0) return 0;
    // co-residency could not be granted: set copy CTAs aside instead (they come first in the
    // grid, so the CTAs that wait for them never keep them from starting)
    cudaGetLastError();
    a.inline_copy = 0;
    a.num_copy_ctas = 16;
  }
  return go(a.num_copy_ctas);
}

}  // namespace gemm
}  // namespace psdev

using namespace psdev;

extern "C" int psdev_gemm_bf16(const void* x, const void* w, void* c, int64_t M, int64_t N,
                               int64_t K, int num_ctas, uint64_t timeout_ns, void* stream) {
  gemm::Args a{};
  a.M = M; a.N = N; a.K = K;
  a.c = static_cast<__nv_bfloat16*>(c);
  a.timeout_ns = timeout_ns ? timeout_ns : 2000000000ull;
  a.fused = 0;
  return gemm::run(a, x, w, num_ctas, (cudaStream_t)stream);
}

// How ring mode moves W: 1 = two threads per CTA, bulk (TMA) loads and stores; 0 = two warps
// per CTA, 16-byte asynchronous copies through the load/store path and bulk stores.  Chunk
// size in elements.  The defaults can be preset with PSB200_PULL_RING=tma|lsu and
// PSB200_PULL_RING_CHUNK=<bytes: 4096, 8192 or 16384>.
static std::atomic<int> g_ring_mode{[] {
  const char* e = getenv("PSB200_PULL_RING");
  return (e && e[0] == 'l') ? 0 : 1;
}()};
static std::atomic<int> g_ring_chunk{[] {
  const char* e = getenv("PSB200_PULL_RING_CHUNK");
  const int v = e ? atoi(e) : 0;
  return (v == 4096 || v == 8192 || v == 16384) ? v / 2 : 4096;
}()};

extern "C" int psdev_pull_ring_config(int mode, int chunk_bytes) {
  if (mode != 0 && mode != 1) return PSDEV_ERR_ARG;
  if (chunk_bytes != 0 && chunk_bytes != 4096 && chunk_bytes != 8192 && chunk_bytes != 16384)
    return PSDEV_ERR_ARG;
  g_ring_mode.store(mode, std::memory_order_relaxed);
  g_ring_chunk.store(chunk_bytes ? chunk_bytes / 2 : 4096, std::memory_order_relaxed);
  return 0;
}

extern "C" int psdev_pull_gemm_bf16(const psdev_world_t* w, const psdev_table_t* t,
                                    int64_t w_elem_off, const void* x, void* c, int64_t M,
                                    int64_t N, int64_t K, int num_copy_ctas, int num_ctas,
                                    uint64_t timeout_ns, void* stream) {
  if (!w || !t || w->world < 1 || w->world > PSDEV_MAX_RANKS) return PSDEV_ERR_ARG;
  if (t->out_dtype != PSDEV_BF16) return PSDEV_ERR_UNSUPPORTED;
  if (w_elem_off < 0 || (w_elem_off & 7) || w_elem_off + N * K > t->n) return PSDEV_ERR_ARG;
  if (w->heap_bytes && (t->weight_off < PSDEV_CTRL_BYTES || t->weight_off > w->heap_bytes ||
                        static_cast<uint64_t>(t->n) * 2 > w->heap_bytes - t->weight_off))
    return PSDEV_ERR_BOUNDS;  // the weight buffer must lie inside the arena
  gemm::Args a{};
  a.M = M; a.N = N; a.K = K;
  a.c = static_cast<__nv_bfloat16*>(c);
  a.timeout_ns = timeout_ns ? timeout_ns : 2000000000ull;
  a.fused = w->world > 1 ? 1 : 0;
  // num_copy_ctas > 0: that many CTAs are set aside for the all-gather; <= 0: ring mode, one
  // thread of every GEMM CTA moves W with bulk copies through shared memory
  if (t->blk <= 0 || (t->blk & 7)) return PSDEV_ERR_ARG;
  const int ring_mode = g_ring_mode.load(std::memory_order_relaxed);
  const int ring_chunk = g_ring_chunk.load(std::memory_order_relaxed);
  a.ring_mode = ring_mode;
  // load/store path: 16 KB of ring per warp, at least two chunks; bulk loads: at most 4 slots
  a.ring_chunk = ring_mode == 0 ? (ring_chunk > 4096 ? 4096 : ring_chunk)
                                : (ring_chunk < 4096 ? 4096 : ring_chunk);
  a.inline_copy = (a.fused && num_copy_ctas <= 0) ? 1 : 0;
  a.num_copy_ctas = a.fused ? (num_copy_ctas > 0 ? num_copy_ctas : 16) : 0;
  for (int p = 0; p < w->world; ++p) a.base[p] = w->peer_base[p];
  a.rank = w->rank;
  a.world = w->world;
  a.weight_off = t->weight_off;
  a.w_elem_off = w_elem_off;
  a.blk = t->blk;
  const char* wl = static_cast<const char*>(w->peer_base[w->rank]) + t->weight_off + w_elem_off * 2;
  return gemm::run(a, x, wl, num_ctas, (cudaStream_t)stream);
}

extern "C" int64_t psdev_pull_plan_chunk(int64_t w_elem_off, int64_t nk, int blk, int world,
                                         int rank, int64_t i, int* owner, int64_t* begin,
                                         int64_t* end) {
  if (nk <= 0 || blk <= 0 || world < 2 || rank < 0 || rank >= world) return 0;
  const gemm::PullPlan pl = gemm::make_pull_plan(w_elem_off, nk, blk, world, rank);
  if (i >= 0 && i < pl.n && owner && begin && end) {
    long long b = 0, e = 0;
    gemm::pull_chunk(pl, i, owner, &b, &e);
    *begin = b;
    *end = e;
  }
  return pl.n;
}

// Selects the kernel variant of later GEMM launches: 128 or 256 (output-tile height of the
// one-CTA kernels), 2 (CTA pairs, tcgen05 cta_group::2), or 0 for the built-in choice by shape.
extern "C" int psdev_gemm_config(int tile_m) {
  if (tile_m != 0 && tile_m != 128 && tile_m != 256 && tile_m != 2) return PSDEV_ERR_ARG;
  gemm::g_tile_m.store(tile_m);
  return 0;
}

// Reads (synchronously) and clears the error word of the GEMM scratch of the current device.
extern "C" int psdev_gemm_status(int32_t* status) {
  int err = 0;
  gemm::Scratch* s = gemm::scratch_for_current_device(&err);
  if (!s) return err;
  cudaError_t e = cudaMemcpy(status, &s->status, sizeof(int32_t), cudaMemcpyDeviceToHost);
  if (e != cudaSuccess) return (int)e;
  if (*status != 0) e = cudaMemset(&s->status, 0, sizeof(int));
  return (int)e;
}

// ================== variant that allocates nothing (see pull_gemm_noalloc.h) ==================
#include <cstdio>

#include "kernels/pull_gemm_noalloc.h"

// Scratch of psdev_gemm_bf16_noalloc.  In host code this name is only a handle for
// cudaGetSymbolAddress: it is not a device address and must never be passed to a kernel.
static __device__ __align__(256) unsigned char g_noalloc_scratch[PSDEV_NOALLOC_SCRATCH_BYTES];
static_assert(sizeof(psdev::gemm::Scratch) <= PSDEV_NOALLOC_SCRATCH_BYTES,
              "static scratch too small for the kernel's counters");

namespace {
// Device address of g_noalloc_scratch on each device, resolved on the first call there.
psdev::gemm::Scratch* g_noalloc_ptr[64] = {};
std::mutex g_noalloc_mu;

int noalloc_scratch(psdev::gemm::Scratch** out) {
  int dev = 0;
  cudaError_t e = cudaGetDevice(&dev);
  if (e != cudaSuccess) return (int)e;
  if (dev < 0 || dev >= 64) return PSDEV_ERR_ARG;
  std::lock_guard<std::mutex> lk(g_noalloc_mu);
  if (!g_noalloc_ptr[dev]) {
    void* p = nullptr;
    e = cudaGetSymbolAddress(&p, g_noalloc_scratch);  // address on the current device
    if (e != cudaSuccess) return (int)e;
    if (!p) return PSDEV_ERR_UNSUPPORTED;
    g_noalloc_ptr[dev] = static_cast<psdev::gemm::Scratch*>(p);
  }
  *out = g_noalloc_ptr[dev];
  return 0;
}
}  // namespace

extern "C" int psdev_gemm_bf16_noalloc(const void* x, const void* w, void* c, int64_t M,
                                       int64_t N, int64_t K, int num_ctas, uint64_t timeout_ns,
                                       int32_t* status_dev, void* stream) {
  using namespace psdev::gemm;
  if (M <= 0 || N <= 0 || K <= 0 || (N & 7) || (K & 7)) return PSDEV_ERR_ARG;
  if (((uintptr_t)x & 15) || ((uintptr_t)w & 15) || ((uintptr_t)c & 15)) return PSDEV_ERR_ARG;
  const int BN = (N % 256 == 0 || N > 1024) ? 256 : 128;
  const int64_t npanels = (N + BN - 1) / BN;
  if (npanels >= kMaxPanels) {
    fprintf(stderr,
            "psdev_gemm_bf16_noalloc: N = %lld needs %lld column panels of %d; the static "
            "scratch of this entry point holds counters for at most %d panels\n",
            (long long)N, (long long)npanels, BN, kMaxPanels - 1);
    return PSDEV_ERR_TOO_LARGE;
  }
  Scratch* scratch = nullptr;
  int rc = noalloc_scratch(&scratch);
  if (rc) return rc;
  cudaStream_t s = (cudaStream_t)stream;
  Args a{};
  a.M = M; a.N = N; a.K = K;
  a.c = static_cast<__nv_bfloat16*>(c);
  a.scratch = scratch;
  a.timeout_ns = timeout_ns ? timeout_ns : 2000000000ull;
  a.fused = 0;
  // everything that can fail on the host comes before the first operation on the stream
  CUtensorMap tx, tw;
  rc = make_tmap(&tx, x, M, K, BM);
  if (rc) return rc;
  rc = make_tmap(&tw, w, N, K, BN);
  if (rc) return rc;
  // the array keeps the previous call's contents: counters and error word start at zero
  cudaError_t e = cudaMemsetAsync(scratch, 0, sizeof(Scratch), s);
  if (e != cudaSuccess) return (int)e;
  int dev = 0, sms = 148;
  cudaGetDevice(&dev);
  cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
  const long long tiles = ((M + BM - 1) / BM) * npanels;
  int grid = num_ctas > 0 ? num_ctas : sms;
  if (tiles < grid) grid = (int)tiles;
  rc = BN == 256 ? launch<256>(a, tx, tw, grid, s) : launch<128>(a, tx, tw, grid, s);
  if (rc) return rc;
  if (status_dev) {
    e = cudaMemcpyAsync(status_dev, &scratch->status, sizeof(int32_t), cudaMemcpyDeviceToDevice, s);
    if (e != cudaSuccess) return (int)e;
  }
  return 0;
}
