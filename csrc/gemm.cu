// bf16 GEMM family for sm_100a: C[M,N] = alpha * A[M,K] * B[N,K]^T (+ C), fp32 accumulation in TMEM.
//
// Persistent, warp-specialised kernel, one CTA per SM:
//   warp 0     TMA producer  (cp.async.bulk.tensor, 128-byte swizzle, no multicast)
//   warp 1     MMA issuer    (tcgen05.mma cta_group::1, M=128, N=BLOCK_N, K=16 per instruction)
//   warps 2-5  epilogue      (tcgen05.ld 32x32b, convert, store; overlaps the next tile's main loop
//                             through two TMEM accumulators)
// Either operand may be K-major (rows of K contiguous) or MN-major (the M/N index contiguous), so
// the three GEMMs of a linear layer (Y = X W^T, dX = dY W, dW = dY^T X) run without a transpose.
// The fp32 output mode with accumulate writes weight gradients straight into a flat fp32 gradient
// buffer (the cast and the micro-batch accumulation of a sharded-data-parallel step).
#include <stdlib.h>
#include <string.h>

#include "common.cuh"
#include "yafsdp_b200.h"

YF_TU_STATUS()

namespace {

constexpr int BLOCK_M = 128;
constexpr int BLOCK_K = 64;   // 64 bf16 = one 128-byte swizzle row
constexpr int UMMA_K = 16;
constexpr int GEMM_THREADS = 192;
constexpr int GATHER_THREADS = 224;  // gather mode: one more warp, for the communication role

// MODE_PLAIN: C is stored locally through TMA.  MODE_SCATTER: GEMM -> reduce-scatter, the fp32 rows of C are pushed to the
// ranks that own them.  MODE_GATHER: all-gather -> GEMM, the kernel also gathers the layer that B is part of (see FusedArgs).
constexpr int MODE_PLAIN = 0, MODE_SCATTER = 1, MODE_GATHER = 2;
constexpr int SCATTER_COLS = 64;                         // columns per pushed row piece: 256 bytes of fp32
constexpr int SCATTER_PITCH = SCATTER_COLS * 4 + 16;     // row pitch of the staging block (16 B of padding: no bank conflicts)

template <int BLOCK_N, int CG, int MODE = MODE_PLAIN>
struct GemmCfg {
  static constexpr int B_ROWS = BLOCK_N / CG;  // rows of B (N extent) in one CTA's shared memory
  static constexpr int A_BYTES = BLOCK_M * BLOCK_K * 2;
  static constexpr int B_BYTES = B_ROWS * BLOCK_K * 2;
  static constexpr int STAGE_BYTES = A_BYTES + B_BYTES;
  static constexpr int RING_BYTES = (MODE == MODE_GATHER) ? 6 * 16384 : 0;  // the communication role's ring (COMM_SLOTS pieces)
  static constexpr int STAGES = (MODE == MODE_SCATTER) ? (STAGE_BYTES == 49152 ? 3 : 4)
                                : (MODE == MODE_GATHER) ? (STAGE_BYTES == 49152 ? 2 : 3)
                                                        : ((STAGE_BYTES == 49152) ? 4 : 6);
  static constexpr int TMEM_COLS = 2 * BLOCK_N;  // two accumulators (power of two: 256 or 512)
  // plain: two [128 rows x 128 B] swizzled blocks for TMA stores; scatter: two [128 rows x 256 B (+ padding)] linear blocks
  static constexpr int STAGING_BYTES = (MODE == MODE_SCATTER) ? 2 * BLOCK_M * SCATTER_PITCH : 2 * 16384 + RING_BYTES;
  static constexpr int SMEM_BYTES = 1024 + STAGES * STAGE_BYTES + STAGING_BYTES + 256;
};

constexpr int MAX_RANKS = 16;
constexpr int MAX_GROUP = 4;  // problems of one grouped launch (the weight-gradient GEMMs of a decoder layer)

struct GemmArgs {
  void* C;
  int M, N, K;
  long long ldc;
  float alpha;
  int a_mn, b_mn, out_f32, accumulate;
  // optional bf16 residual [M, N] with row pitch ldr, added in fp32 before the bf16 output is rounded (bf16 output, plain
  // mode): a block's "x + proj(...)" costs no pass of its own over the activations
  const void* R;
  long long ldr;
  // Grouped launch (scatter mode): n_prob problems that share K and the operand majors, in the order of their positions in
  // the flat layer gradient.  Tiles are numbered problem by problem, rows first (= in flat order); tile_prefix[p] = number
  // of tiles in front of problem p; own_start[o] = first tile whose rows begin in the shard of rank o.  The launch deals the
  // owners' tiles round-robin, starting with the rank after this one: step t works on tile t / world of owner
  // (rank + 1 + t % world) % world, so every rank pushes to all owners (and computes for itself) all the time and no
  // owner's NVLink ingress becomes a hot spot whatever the skew between the ranks.  n_prob == 0: one problem, M x N above.
  int n_prob;
  int Mp[MAX_GROUP], Np[MAX_GROUP];
  long long flat_off[MAX_GROUP];
  int tile_prefix[MAX_GROUP + 1];
  int own_start[MAX_RANKS + 1];
  int steps;   // world * (largest number of tiles of one owner)
};

// operand tensor maps of up to MAX_GROUP problems (entry 0 alone for an ordinary launch)
struct GroupMaps {
  CUtensorMap a[MAX_GROUP], b[MAX_GROUP];
};

// Arguments of the two fused compute + collective modes (both off when zero-initialised).
//
// gather (all-gather -> GEMM, MODE_GATHER): every CTA of the GEMM carries one extra warp whose elected thread pulls its
// share of every rank's bf16 shard of the layer (bulk loads from peer memory over NVLink into a small ring in shared
// memory, bulk stores from there into the local layer buffer) and, for every piece that lies inside B, adds the piece's
// bytes to the counter of the B column block it belongs to.  The producer warps wait (bounded) until the counter of a tile's
// column block says that all of its rows have landed, then load B from the local buffer as usual.  The GEMM therefore
// runs while the layer is still arriving, no SM is given up to communication, and when the kernel ends the whole layer
// buffer is gathered for the GEMMs that follow.
//
// scatter (GEMM -> reduce-scatter, MODE_SCATTER): the fp32 epilogue does not store C locally; every row piece goes to the
// rank that owns its position of the flat layer gradient, into that owner's slot for this rank (slot r of the owner's
// reduce buffer = contributions of rank r to the owner's shard).  The owner then sums its `world` slots locally in rank
// order.
struct FusedArgs {
  // gather
  int gather;
  int world, rank;
  unsigned long long* counters;      // [number of B column blocks] bytes landed, monotonic over calls (device memory of this GPU)
  unsigned long long epoch;          // this call completes a block when its counter reaches epoch * bytes of the block
  const void* peer_in[MAX_RANKS];
  uint8_t* layer_buf;
  long long shard_bytes, b_byte_off;
  // optional: sum of squares of the (alpha-scaled) fp32 output, atomically added to *sumsq (gradient-norm fusion)
  float* sumsq;
  // scatter
  int scatter;
  int wire_bf16;                     // the slots hold bf16 (the owner accumulates in fp32); else fp32
  void* peer_grad[MAX_RANKS];
  long long c_flat_off, shard_numel;
};

YF_DEVINL unsigned long long ld_relaxed_gpu_u64(const unsigned long long* p) {
  unsigned long long v;
  asm volatile("ld.relaxed.gpu.global.u64 %0, [%1];" : "=l"(v) : "l"(p) : "memory");
  return v;
}
YF_DEVINL void red_add_relaxed_gpu_u64(unsigned long long* p, unsigned long long v) {
  asm volatile("red.relaxed.gpu.global.add.u64 [%0], %1;" ::"l"(p), "l"(v) : "memory");
}
YF_DEVINL void fence_proxy_async_global() { asm volatile("fence.proxy.async.global;" ::: "memory"); }

YF_DEVINL void bulk_load(void* smem_dst, const void* gsrc, uint32_t bytes, uint64_t* bar) {
  asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::"r"(smem_u32(smem_dst)),
               "l"(reinterpret_cast<uint64_t>(gsrc)), "r"(bytes), "r"(smem_u32(bar))
               : "memory");
}
YF_DEVINL void bulk_store(void* gdst, const void* smem_src, uint32_t bytes) {
  asm volatile("cp.async.bulk.global.shared::cta.bulk_group [%0], [%1], %2;" ::"l"(reinterpret_cast<uint64_t>(gdst)),
               "r"(smem_u32(smem_src)), "r"(bytes)
               : "memory");
}
YF_DEVINL void tma_store_wait1() { asm volatile("cp.async.bulk.wait_group 1;" ::: "memory"); }

// Communication role of the gather mode: ONE thread of every CTA.  Piece q of the layer (q = 0, 1, ...) is piece q / world
// of the shard of rank (rank + q % world) % world, so consecutive pieces come from different owners and, at any moment, the
// ranks read from different peers; CTA c moves the pieces c, c + grid, c + 2 grid, ...  A piece goes peer -> ring slot
// (bulk load, completion on an mbarrier) -> local layer buffer (bulk store); four loads and two stores are in flight.
constexpr int COMM_PIECE = 16384;
constexpr int COMM_SLOTS = 6;
constexpr int COMM_AHEAD = 4;   // loads in flight per CTA (64 KB; x 148 CTAs covers the NVLink bandwidth-delay product with margin)

__device__ void gather_comm_role(const FusedArgs& fa, long long b_bytes, long long block_bytes, uint8_t* ring, uint64_t* ring_bars) {
  const long long pps = (fa.shard_bytes + COMM_PIECE - 1) / COMM_PIECE;  // pieces per shard
  const long long total = pps * fa.world;
  const long long first = blockIdx.x, step = gridDim.x;
  const long long mine = first < total ? (total - first + step - 1) / step : 0;
  auto piece = [&](long long i, const uint8_t*& src, long long& layer_off, uint32_t& bytes) {
    const long long q = first + i * step;
    const int owner = (fa.rank + (int)(q % fa.world)) % fa.world;
    const long long lo = (q / fa.world) * COMM_PIECE;
    bytes = (uint32_t)min((long long)COMM_PIECE, fa.shard_bytes - lo);
    src = reinterpret_cast<const uint8_t*>(fa.peer_in[owner]) + lo;
    layer_off = (long long)owner * fa.shard_bytes + lo;
  };
  auto issue_load = [&](long long i) {
    const uint8_t* src; long long off; uint32_t bytes;
    piece(i, src, off, bytes);
    const int slot = (int)(i % COMM_SLOTS);
    mbar_expect_tx(&ring_bars[slot], bytes);
    bulk_load(ring + slot * COMM_PIECE, src, bytes, &ring_bars[slot]);
  };
  // piece i has been written to the layer buffer: credit the B column blocks it overlaps
  auto publish = [&](long long i) {
    const uint8_t* src; long long off; uint32_t bytes;
    piece(i, src, off, bytes);
    long long lo = max(off, fa.b_byte_off) - fa.b_byte_off, hi = min(off + (long long)bytes, fa.b_byte_off + b_bytes) - fa.b_byte_off;
    if (lo >= hi) return;
    // The piece's bulk store has completed (wait_group): its bytes have been written at the L2, the point where the
    // counter's atomic add is performed too, so the add cannot be seen before them.  No fence here: a release fence or a
    // proxy fence waits for everything this SM has in flight (the GEMM's own loads, stores and MMAs), tens of microseconds
    // per piece while the GEMM runs; the reader acquires and fences once per tile instead.
    while (lo < hi) {
      const long long blk = lo / block_bytes;
      const long long end = min(hi, (blk + 1) * block_bytes);
      red_add_relaxed_gpu_u64(fa.counters + blk, (unsigned long long)(end - lo));
      lo = end;
    }
  };
  for (long long i = 0; i < COMM_AHEAD && i < mine; ++i) issue_load(i);
  long long done = 0, stored = 0;  // pieces published / pieces whose store has been issued
#ifdef YF_GATHER_PROFILE
  unsigned long long tp[5] = {0, 0, 0, 0, 0};
  unsigned long long t_a = yf_globaltimer(), t_b;
#define YF_TICK(k) t_b = yf_globaltimer(); tp[k] += t_b - t_a; t_a = t_b;
#else
#define YF_TICK(k)
#endif
  for (long long i = 0; i < mine; ++i, ++stored) {
    const int slot = (int)(i % COMM_SLOTS);
    if (!mbar_wait(&ring_bars[slot], (uint32_t)((i / COMM_SLOTS) & 1), 12)) break;  // gave up: nothing more is copied or published
    YF_TICK(0)
    const uint8_t* src; long long off; uint32_t bytes;
    piece(i, src, off, bytes);
    bulk_store(fa.layer_buf + off, ring + slot * COMM_PIECE, bytes);
    tma_store_commit();
    tma_store_wait_read1();  // every store but this one has finished reading its slot: the slot of piece i - 2 is free
    YF_TICK(1)
    if (i + COMM_AHEAD < mine) issue_load(i + COMM_AHEAD);  // into slot (i + 4) % 6 == (i - 2) % 6
    YF_TICK(2)
    tma_store_wait1();       // every store but this one has completed: piece i - 1 is in the layer buffer
    YF_TICK(3)
    if (i >= 1) { publish(i - 1); done = i; }
    YF_TICK(4)
  }
#ifdef YF_GATHER_PROFILE
  for (int k = 0; k < 5; ++k) fa.counters[1024 + 8 * blockIdx.x + k] = tp[k];
  fa.counters[1024 + 8 * blockIdx.x + 5] = (unsigned long long)mine;
#endif
  tma_store_wait0();
  for (long long i = done; i < stored; ++i) publish(i);
}

template <int BLOCK_N, int CG, int MODE>
__global__ void __launch_bounds__(MODE == MODE_GATHER ? GATHER_THREADS : GEMM_THREADS, 1)
gemm_bf16_tcgen05_kernel(const __grid_constant__ GroupMaps maps, const __grid_constant__ CUtensorMap tma_c, GemmArgs args, FusedArgs fa) {
  using Cfg = GemmCfg<BLOCK_N, CG, MODE>;
  // CG == 2: the grid is a sequence of CTA pairs (clusters of two); a pair works on one 256 x BLOCK_N tile, CTA `crank` of
  // the pair on its rows [crank * 128, +128) with the B rows [crank * BLOCK_N / 2, +BLOCK_N / 2) in its shared memory
  const uint32_t crank = (CG == 2) ? cluster_ctarank() : 0u;
  const bool leader = crank == 0;
  const int unit = (int)blockIdx.x / CG;        // index among the tile workers (CTAs or pairs)
  const int nunits = (int)gridDim.x / CG;
  constexpr int STAGES = Cfg::STAGES;
  constexpr int TILE_M = BLOCK_M * CG;
  constexpr int B_ROWS = Cfg::B_ROWS;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint8_t* staging = smem + STAGES * Cfg::STAGE_BYTES;
  uint64_t* bars = reinterpret_cast<uint64_t*>(staging + Cfg::STAGING_BYTES);
  uint64_t* full = bars;                 // [STAGES]  (pairs: only the leader's are used, both CTAs' loads count there)
  uint64_t* empty = bars + STAGES;       // [STAGES]
  uint64_t* tfull = bars + 2 * STAGES;   // [2]
  uint64_t* tempty = tfull + 2;          // [2]       (pairs: only the leader's are used)
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(tempty + 2);
  uint64_t* ring_bars = reinterpret_cast<uint64_t*>(tmem_slot + 2);   // [COMM_SLOTS], gather mode
  uint8_t* ring = staging + Cfg::STAGING_BYTES - Cfg::RING_BYTES;     // gather mode: the tail of the staging area

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const int K = args.K;
  const int num_m = (args.M + TILE_M - 1) / TILE_M;
  const int num_n = (args.N + BLOCK_N - 1) / BLOCK_N;
  const int num_k = (K + BLOCK_K - 1) / BLOCK_K;
  const bool grouped = (MODE == MODE_SCATTER) && args.n_prob > 0;
  const int num_tiles = grouped ? args.steps : num_m * num_n;  // steps of the tile loop (a grouped step may be empty)
  constexpr int GROUP_M = 16 / CG;  // 2048 rows of A share a column block of B through L2

  if (threadIdx.x == 0) {
    tma_prefetch_desc(&maps.a[0]);
    tma_prefetch_desc(&maps.b[0]);
    tma_prefetch_desc(&tma_c);
    for (int s = 0; s < STAGES; ++s) {
      mbar_init(&full[s], 1);
      mbar_init(&empty[s], 1);
    }
    for (int a = 0; a < 2; ++a) {
      mbar_init(&tfull[a], 1);
      mbar_init(&tempty[a], 4 * CG);  // one arrival per epilogue warp of every CTA of the pair
    }
    if (MODE == MODE_GATHER)
      for (int i = 0; i < COMM_SLOTS; ++i) mbar_init(&ring_bars[i], 1);
    mbar_fence_init();
  }
  if (warp == 1) {
    if (CG == 2) {
      tmem_alloc_pair(tmem_slot, Cfg::TMEM_COLS);
      tmem_relinquish_pair();
    } else {
      tmem_alloc(tmem_slot, Cfg::TMEM_COLS);
      tmem_relinquish();
    }
  }
  tc_fence_before();
  __syncthreads();
  if (CG == 2) cluster_sync_all();  // the peer's barriers and TMEM exist before anything is sent to them
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;

  // step t of this launch -> problem p, first row m0 (of this CTA) and first column n0 of the tile; false: empty step
  auto tile_coords = [&](int t, int& p, int& m0, int& n0) -> bool {
    if (grouped) {
      const int o = (fa.rank + 1 + t % fa.world) % fa.world;
      const int g = args.own_start[o] + t / fa.world;
      if (g >= args.own_start[o + 1]) return false;  // this owner has fewer tiles than the largest one
      p = 0;
      while (p + 1 < args.n_prob && g >= args.tile_prefix[p + 1]) ++p;
      const int local = g - args.tile_prefix[p];
      const int nn = (args.Np[p] + BLOCK_N - 1) / BLOCK_N;
      m0 = (local / nn) * TILE_M + (int)crank * BLOCK_M;
      n0 = (local % nn) * BLOCK_N;
      return true;
    }
    p = 0;
    const int per_group = GROUP_M * num_n;
    const int g = t / per_group;
    const int first_m = g * GROUP_M;
    const int gsize = min(GROUP_M, num_m - first_m);
    const int r = t - g * per_group;
    m0 = (first_m + r % gsize) * TILE_M + (int)crank * BLOCK_M;
    n0 = (r / gsize) * BLOCK_N;
    return true;
  };

  if (warp == 0) {
    // ------------------------------------------------------------ TMA producer (one per CTA)
    if (lane == 0) {
      uint32_t it = 0;
      bool alive = true;
      for (int t = unit; t < num_tiles && alive; t += nunits) {
        int p, m0, n0;
        if (!tile_coords(t, p, m0, n0)) continue;
        const CUtensorMap* tma_a = &maps.a[p];
        const CUtensorMap* tma_b = &maps.b[p];
        const int N = grouped ? args.Np[p] : args.N;
        if (MODE == MODE_GATHER) {
          // the rows [n0, n0 + BLOCK_N) of B must have landed in the local layer buffer: the column block's counter says so
          const int blk = n0 / BLOCK_N;
          const unsigned long long want = fa.epoch * (unsigned long long)((long long)min(BLOCK_N, N - n0) * K * 2);
          // Poll with relaxed loads and pauses: an acquire per poll is a memory fence per poll, and such a fence waits for
          // everything the busy SM has in flight (tens of microseconds) and holds up the communication warp next door.
          // The rows were written by bulk stores (asynchronous proxy) of CTAs of this GPU and are read by TMA (the same
          // proxy) straight from the L2, where they were complete before the counter moved; the TMA loads are issued after
          // the poll has returned.  So no acquire and no proxy fence follow: either one waits for the communication warp's
          // copies in flight, which never pause (measured: 1.7 ms instead of 0.34 ms for the kernel).
          const uint64_t t0 = yf_globaltimer();
          for (uint32_t spin = 0; ld_relaxed_gpu_u64(fa.counters + blk) < want; ++spin) {
            __nanosleep(400);
            if ((spin & 63u) == 63u && (yf_aborted() || yf_globaltimer() - t0 > YF_WAIT_NS_DEFAULT)) {
              yf_raise(YF_ERR_FLAG_TIMEOUT, 11);
              alive = false;
              break;
            }
          }
          if (!alive) break;
        }
        const int nb = n0 + (int)crank * B_ROWS;  // first B row this CTA holds
        for (int kb = 0; kb < num_k; ++kb, ++it) {
          const int s = it % STAGES;
          const uint32_t ph = (it / STAGES) & 1;
          if (!mbar_wait(&empty[s], ph ^ 1, 10)) { alive = false; break; }
          uint8_t* sa = smem + s * Cfg::STAGE_BYTES;
          uint8_t* sb = sa + Cfg::A_BYTES;
          const int k0 = kb * BLOCK_K;
          if (CG == 2) {
            // both CTAs' bytes are counted on the leader's barrier (the thread that issues the MMAs waits there)
            if (leader) mbar_expect_tx(&full[s], 2 * Cfg::STAGE_BYTES);
            const uint32_t fb = mapa_shared(smem_u32(&full[s]), 0);
            if (!args.a_mn) {
              tma_load_2d_pair(sa, tma_a, fb, k0, m0);
            } else {
#pragma unroll
              for (int j = 0; j < BLOCK_M / 64; ++j) tma_load_2d_pair(sa + j * (BLOCK_K * 128), tma_a, fb, m0 + j * 64, k0);
            }
            if (!args.b_mn) {
              tma_load_2d_pair(sb, tma_b, fb, k0, nb);
            } else {
#pragma unroll
              for (int j = 0; j < B_ROWS / 64; ++j) tma_load_2d_pair(sb + j * (BLOCK_K * 128), tma_b, fb, nb + j * 64, k0);
            }
          } else {
            mbar_expect_tx(&full[s], Cfg::STAGE_BYTES);
            if (!args.a_mn) {
              tma_load_2d(sa, tma_a, &full[s], k0, m0);
            } else {
#pragma unroll
              for (int j = 0; j < BLOCK_M / 64; ++j) tma_load_2d(sa + j * (BLOCK_K * 128), tma_a, &full[s], m0 + j * 64, k0);
            }
            if (!args.b_mn) {
              tma_load_2d(sb, tma_b, &full[s], k0, nb);
            } else {
#pragma unroll
              for (int j = 0; j < B_ROWS / 64; ++j) tma_load_2d(sb + j * (BLOCK_K * 128), tma_b, &full[s], nb + j * 64, k0);
            }
          }
        }
      }
      if (!alive) {
        // give copies already in flight a bounded time to land before the CTA may exit
        const uint64_t t0 = yf_globaltimer();
        while (yf_globaltimer() - t0 < 200000ull) __nanosleep(1000);
      }
    }
  } else if (warp == 1) {
    // ------------------------------------------------------------ MMA issuer (pairs: the leader CTA issues for both)
    if (lane == 0 && leader) {
      const uint32_t idesc = umma_idesc_bf16(TILE_M, BLOCK_N, args.a_mn, args.b_mn);
      const uint32_t a_lbo = args.a_mn ? BLOCK_K * 128 : 0, b_lbo = args.b_mn ? BLOCK_K * 128 : 0;
      const uint32_t a_kstep = args.a_mn ? UMMA_K * 128 : UMMA_K * 2, b_kstep = args.b_mn ? UMMA_K * 128 : UMMA_K * 2;
      uint32_t it = 0;
      bool alive = true;
      int lt = 0;
      for (int t = unit; t < num_tiles && alive; t += nunits) {
        {
          int p, m0, n0;
          if (!tile_coords(t, p, m0, n0)) continue;
        }
        const int acc = lt & 1;
        const uint32_t acc_ph = (lt >> 1) & 1;
        ++lt;
        if (!mbar_wait(&tempty[acc], acc_ph ^ 1, 20)) { alive = false; break; }
        tc_fence_after();
        const uint32_t d_tmem = tmem_base + acc * BLOCK_N;
        for (int kb = 0; kb < num_k; ++kb, ++it) {
          const int s = it % STAGES;
          const uint32_t ph = (it / STAGES) & 1;
          if (!mbar_wait(&full[s], ph, 21)) { alive = false; break; }
          tc_fence_after();
          const uint32_t sa = smem_u32(smem + s * Cfg::STAGE_BYTES);
          const uint32_t sb = sa + Cfg::A_BYTES;
#pragma unroll
          for (int k = 0; k < BLOCK_K / UMMA_K; ++k) {
            const uint64_t adesc = umma_smem_desc_sw128(sa + k * a_kstep, a_lbo, 1024);
            const uint64_t bdesc = umma_smem_desc_sw128(sb + k * b_kstep, b_lbo, 1024);
            if (CG == 2) tc_mma_bf16_pair(d_tmem, adesc, bdesc, idesc, (kb | k) != 0 ? 1u : 0u);
            else tc_mma_bf16(d_tmem, adesc, bdesc, idesc, (kb | k) != 0 ? 1u : 0u);
          }
          // frees the stage (in both CTAs of a pair) once these MMAs have read it
          if (CG == 2) {
            const uint32_t eb = smem_u32(&empty[s]);
            tc_commit_pair(mapa_shared(eb, 0));
            tc_commit_pair(mapa_shared(eb, 1));
          } else {
            tc_commit(&empty[s]);
          }
        }
        if (alive) {
          if (CG == 2) {
            const uint32_t tb = smem_u32(&tfull[acc]);
            tc_commit_pair(mapa_shared(tb, 0));
            tc_commit_pair(mapa_shared(tb, 1));
          } else {
            tc_commit(&tfull[acc]);
          }
        }
      }
    }
  } else if (MODE == MODE_GATHER && warp == 6) {
    // ------------------------------------------------------------ communication role (gather mode)
    if (lane == 0) gather_comm_role(fa, (long long)args.N * K * 2, (long long)BLOCK_N * K * 2, ring, ring_bars);
  } else {
    // ------------------------------------------------------------ epilogue (4 warps = 128 TMEM lanes)
    // TMEM -> registers -> 128-byte-swizzled staging block in shared memory -> TMA store (or TMA
    // reduce-add when accumulating): full 128-byte lines leave the SM, edges are clipped by the TMA unit.
    const int q = warp & 3;  // a warp may only touch TMEM lanes [32*(warp%4), +32)
    const int r_in_tile = q * 32 + lane;
    const bool store_thread = (threadIdx.x == 64);
    const int cols_per_chunk = args.out_f32 ? 32 : 64;
    const int n_chunks = BLOCK_N / cols_per_chunk;
    bool alive = true;
    int lt = 0;
    uint32_t chunk_ctr = 0;
    float ss = 0.f;  // sum of squares of this thread's outputs (rows / columns past the edges are exact zeros)
    for (int t = unit; t < num_tiles && alive; t += nunits) {
      int p, m0, n0;
      if (!tile_coords(t, p, m0, n0)) continue;
      const int M = grouped ? args.Mp[p] : args.M, N = grouped ? args.Np[p] : args.N;
      const long long c_flat_off = grouped ? args.flat_off[p] : fa.c_flat_off;
      const int acc = lt & 1;
      const uint32_t acc_ph = (lt >> 1) & 1;
      ++lt;
      const bool gave_up = !mbar_wait(&tfull[acc], acc_ph, 30);
      if (MODE == MODE_SCATTER) {
        if (!__all_sync(0xffffffffu, !gave_up)) { alive = false; break; }  // per-warp epilogue: a warp leaves as a whole
      } else if (named_bar_or(1, 128, gave_up)) {  // the four warps share named barriers below: they leave together
        alive = false;
        break;
      }
      tc_fence_after();
      const uint32_t taddr = tmem_base + ((uint32_t)(q * 32) << 16) + acc * BLOCK_N;
      const float alpha = args.alpha;
      if constexpr (MODE == MODE_SCATTER) {
        // GEMM -> reduce-scatter.  Every thread owns one row of the accumulator: it moves 64 columns at a time from its
        // TMEM lane into its own row of a staging block and sends that 256-byte piece with one bulk store (two where the
        // piece straddles a shard boundary) to the slot that the owning rank keeps for this rank.  No thread touches
        // another thread's row, so the epilogue needs no block-level barrier; bulk groups are per thread.
        // Wire format fp32 (64 columns per piece) or bf16 (128 columns per piece; the owner still accumulates in fp32).
        const int m = m0 + r_in_tile;
        const int esz = fa.wire_bf16 ? 2 : 4;
        const int piece_cols = fa.wire_bf16 ? 2 * SCATTER_COLS : SCATTER_COLS;
        const int n_pieces = BLOCK_N / piece_cols;
        const long long align_mask = fa.wire_bf16 ? 7 : 3;  // 16-byte pieces
#pragma unroll 1
        for (int c = 0; c < n_pieces; ++c, ++chunk_ctr) {
          uint8_t* srow = staging + (chunk_ctr & 1) * (BLOCK_M * SCATTER_PITCH) + r_in_tile * SCATTER_PITCH;
          tma_store_wait_read1();  // the store that read this row two pieces ago has finished reading
          if (fa.wire_bf16) {
#pragma unroll
            for (int quarter = 0; quarter < 4; ++quarter) {
              uint32_t r[32];
              tmem_ld32(taddr + c * piece_cols + quarter * 32, r);
              tmem_ld_wait();
#pragma unroll
              for (int j = 0; j < 4; ++j) {
                uint4 o;
                o.x = pack_bf16x2(alpha * __uint_as_float(r[8 * j + 0]), alpha * __uint_as_float(r[8 * j + 1]));
                o.y = pack_bf16x2(alpha * __uint_as_float(r[8 * j + 2]), alpha * __uint_as_float(r[8 * j + 3]));
                o.z = pack_bf16x2(alpha * __uint_as_float(r[8 * j + 4]), alpha * __uint_as_float(r[8 * j + 5]));
                o.w = pack_bf16x2(alpha * __uint_as_float(r[8 * j + 6]), alpha * __uint_as_float(r[8 * j + 7]));
                *reinterpret_cast<uint4*>(srow + quarter * 64 + j * 16) = o;
              }
            }
          } else {
#pragma unroll
            for (int half = 0; half < 2; ++half) {
              uint32_t r[32];
              tmem_ld32(taddr + c * piece_cols + half * 32, r);
              tmem_ld_wait();
#pragma unroll
              for (int j = 0; j < 8; ++j) {
                float4 o;
                o.x = alpha * __uint_as_float(r[4 * j + 0]);
                o.y = alpha * __uint_as_float(r[4 * j + 1]);
                o.z = alpha * __uint_as_float(r[4 * j + 2]);
                o.w = alpha * __uint_as_float(r[4 * j + 3]);
                *reinterpret_cast<float4*>(srow + half * 128 + j * 16) = o;
              }
            }
          }
          if (c == n_pieces - 1) {  // accumulator fully read: hand it back to the MMA warp (of the leader CTA)
            tc_fence_before();
            __syncwarp();
            if (lane == 0) {
              if (CG == 2) mbar_arrive_cluster(mapa_shared(smem_u32(&tempty[acc]), 0));
              else mbar_arrive(&tempty[acc]);
            }
          }
          fence_proxy_async_smem();
          const int col = n0 + c * piece_cols;
          if (m < M && col < N) {
            const long long ncols = min(piece_cols, N - col);
            const long long f = c_flat_off + (long long)m * N + col;      // position in the flat layer gradient
            const long long o = f / fa.shard_numel;                       // owner rank
            const long long loc = f - o * fa.shard_numel;
            const long long first = min(ncols, fa.shard_numel - loc);
#ifdef YF_DEBUG_BOUNDS
            // debug build: a piece that would leave the owners' slots is recorded and skipped instead of stored
            if (f < 0 || o >= fa.world || (first < ncols && o + 1 >= fa.world) || loc < 0 || (first & align_mask) || (loc & align_mask)) {
              yf_raise(YF_ERR_BAD_ARGUMENT, 40);
              tma_store_commit();
              continue;
            }
#endif
            (void)align_mask;
            uint8_t* dst = reinterpret_cast<uint8_t*>(fa.peer_grad[o]) + ((long long)fa.rank * fa.shard_numel + loc) * esz;
            bulk_store(dst, srow, (uint32_t)(first * esz));
            if (first < ncols) {
              uint8_t* dst2 = reinterpret_cast<uint8_t*>(fa.peer_grad[o + 1]) + (long long)fa.rank * fa.shard_numel * esz;
              bulk_store(dst2, srow + first * esz, (uint32_t)((ncols - first) * esz));
            }
          }
          tma_store_commit();
        }
      } else {
#pragma unroll 1
      for (int c = 0; c < n_chunks; ++c, ++chunk_ctr) {
        uint8_t* stg = staging + (chunk_ctr & 1) * 16384;
        uint8_t* srow = stg + r_in_tile * 128;
        if (store_thread) tma_store_wait_read1();  // the store that last read this block has finished reading
        named_bar_sync(1, 128);
        if (args.out_f32) {
          uint32_t r[32];
          tmem_ld32(taddr + c * 32, r);
          tmem_ld_wait();
#pragma unroll
          for (int j = 0; j < 8; ++j) {
            float4 o;
            o.x = alpha * __uint_as_float(r[4 * j + 0]);
            o.y = alpha * __uint_as_float(r[4 * j + 1]);
            o.z = alpha * __uint_as_float(r[4 * j + 2]);
            o.w = alpha * __uint_as_float(r[4 * j + 3]);
            ss += o.x * o.x + o.y * o.y + o.z * o.z + o.w * o.w;
            *reinterpret_cast<float4*>(srow + ((j ^ (r_in_tile & 7)) << 4)) = o;
          }
        } else {
#pragma unroll
          for (int half = 0; half < 2; ++half) {
            // the residual of this thread's row: 4 x 16 bytes, requested before the accumulator is read (N % 8 == 0)
            uint4 res[4] = {};
            if (args.R != nullptr) {
              const int row = m0 + r_in_tile, col = n0 + c * 64 + half * 32;
              if (row < M) {
                const uint4* rp = reinterpret_cast<const uint4*>(static_cast<const __nv_bfloat16*>(args.R) + (long long)row * args.ldr + col);
#pragma unroll
                for (int j = 0; j < 4; ++j)
                  if (col + 8 * j < N) res[j] = __ldg(rp + j);
              }
            }
            uint32_t r[32];
            tmem_ld32(taddr + c * 64 + half * 32, r);
            tmem_ld_wait();
#pragma unroll
            for (int j = 0; j < 4; ++j) {
              const uint32_t rw[4] = {res[j].x, res[j].y, res[j].z, res[j].w};
              uint32_t ow[4];
#pragma unroll
              for (int w = 0; w < 4; ++w)  // a bf16 pair: low half = even column
                ow[w] = pack_bf16x2(fmaf(alpha, __uint_as_float(r[8 * j + 2 * w]), __uint_as_float(rw[w] << 16)),
                                    fmaf(alpha, __uint_as_float(r[8 * j + 2 * w + 1]), __uint_as_float(rw[w] & 0xffff0000u)));
              *reinterpret_cast<uint4*>(srow + (((half * 4 + j) ^ (r_in_tile & 7)) << 4)) = make_uint4(ow[0], ow[1], ow[2], ow[3]);
            }
          }
        }
        if (c == n_chunks - 1) {  // accumulator fully read: hand it back to the MMA warp (of the leader CTA)
          tc_fence_before();
          __syncwarp();
          if (lane == 0) {
            if (CG == 2) mbar_arrive_cluster(mapa_shared(smem_u32(&tempty[acc]), 0));
            else mbar_arrive(&tempty[acc]);
          }
        }
        fence_proxy_async_smem();
        named_bar_sync(1, 128);
        if (store_thread) {
          const int x = n0 + c * cols_per_chunk;
          if (x < N && m0 < M) {
            if (args.accumulate) tma_reduce_add_2d(&tma_c, stg, x, m0);
            else tma_store_2d(&tma_c, stg, x, m0);
          }
          tma_store_commit();
        }
      }
      }
    }
    if (MODE == MODE_SCATTER || store_thread) tma_store_wait0();  // all of this thread's stores have completed
    if (fa.sumsq != nullptr) {
      ss = warp_sum(ss);
      if (lane == 0) atomicAdd(fa.sumsq, ss);
    }
  }

  tc_fence_before();
  __syncthreads();
  if (CG == 2) cluster_sync_all();  // neither CTA leaves while the other may still read its shared memory or signal its barriers
  if (warp == 1) {
    tc_fence_after();
    if (CG == 2) tmem_dealloc_pair(tmem_base, Cfg::TMEM_COLS);
    else tmem_dealloc(tmem_base, Cfg::TMEM_COLS);
  }
}

// cudaFuncSetAttribute is per device: remember which devices have the opt-in to large dynamic shared memory
template <typename KernelT>
int ensure_smem_optin(KernelT kernel, int bytes, bool (&done)[64]) {
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return -1;
  if (!done[dev]) {
    cudaError_t e = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, bytes);
    if (e != cudaSuccess) return -(int)e;
    done[dev] = true;
  }
  return 0;
}

// One problem's operands (a grouped launch passes several).
struct Operands {
  const void* A;
  const void* B;
  long long lda, ldb;
  int M, N;
};

template <int BLOCK_N, int CG, int MODE = MODE_PLAIN>
int launch_gemm(const Operands* ops, int n_ops, GemmArgs args, const FusedArgs& fa, int sm_limit, cudaStream_t stream) {
  using Cfg = GemmCfg<BLOCK_N, CG, MODE>;
  if (n_ops < 1 || n_ops > MAX_GROUP) return -1;
  GroupMaps maps;
  memset(&maps, 0, sizeof(maps));
  for (int i = 0; i < n_ops; ++i) {
    const Operands& o = ops[i];
    const CUtensorMap* ma = args.a_mn ? yf_tensor_map_2d(o.A, o.M, args.K, o.lda, 64, BLOCK_K, 2, 1)
                                      : yf_tensor_map_2d(o.A, args.K, o.M, o.lda, BLOCK_K, BLOCK_M, 2, 1);
    const CUtensorMap* mb = args.b_mn ? yf_tensor_map_2d(o.B, o.N, args.K, o.ldb, 64, BLOCK_K, 2, 1)
                                      : yf_tensor_map_2d(o.B, args.K, o.N, o.ldb, BLOCK_K, Cfg::B_ROWS, 2, 1);
    if (!ma || !mb) return -2;
    maps.a[i] = *ma;
    maps.b[i] = *mb;
  }
  for (int i = n_ops; i < MAX_GROUP; ++i) {  // unused entries hold a valid descriptor all the same
    maps.a[i] = maps.a[0];
    maps.b[i] = maps.b[0];
  }
  const CUtensorMap* mc = yf_tensor_map_2d(args.C, args.N, args.M, args.ldc, args.out_f32 ? 32 : 64, BLOCK_M, args.out_f32 ? 4 : 2, 1);
  if (!mc) return -2;
  static bool optin[64] = {};
  if (int rc = ensure_smem_optin(gemm_bf16_tcgen05_kernel<BLOCK_N, CG, MODE>, Cfg::SMEM_BYTES, optin)) return rc;
  if (int rc = yf_tu_bind_status()) return rc;
  const int tile_m = BLOCK_M * CG;
  int num_tiles = 0;
  if (args.n_prob > 0) {
    for (int i = 0; i < args.n_prob; ++i) {
      args.tile_prefix[i] = num_tiles;
      num_tiles += ((args.Mp[i] + tile_m - 1) / tile_m) * ((args.Np[i] + BLOCK_N - 1) / BLOCK_N);
    }
    args.tile_prefix[args.n_prob] = num_tiles;
    // own_start[o]: first tile (in flat order) whose rows begin in the shard of rank o or later
    int g = 0, o = 0, most = 0;
    args.own_start[0] = 0;
    for (int i = 0; i < args.n_prob; ++i) {
      const int nn = (args.Np[i] + BLOCK_N - 1) / BLOCK_N, nm = (args.Mp[i] + tile_m - 1) / tile_m;
      for (int m = 0; m < nm; ++m, g += nn) {
        const long long owner = (args.flat_off[i] + (long long)m * tile_m * args.Np[i]) / fa.shard_numel;
        while (o < owner && o < fa.world - 1) args.own_start[++o] = g;
      }
    }
    while (o < MAX_RANKS) args.own_start[++o] = num_tiles;
    for (int r = 0; r < fa.world; ++r) most = most > args.own_start[r + 1] - args.own_start[r] ? most : args.own_start[r + 1] - args.own_start[r];
    args.steps = most * fa.world;
    num_tiles = args.steps;
  } else {
    num_tiles = ((args.M + tile_m - 1) / tile_m) * ((args.N + BLOCK_N - 1) / BLOCK_N);
  }
  int sms = yf_num_sms();
  if (sm_limit > 0 && sm_limit < sms) sms = sm_limit;
  int units = sms / CG;
  if (units < 1) return -1;
  // never more CTAs than SMs (producers may wait on other CTAs' communication warps: all of them must be resident); the
  // gather mode keeps every SM's communication warp even when the GEMM has fewer tiles than that
  if (num_tiles < units && MODE != MODE_GATHER) units = num_tiles;
  const int grid = units * CG;
  cudaLaunchConfig_t cfg;
  memset(&cfg, 0, sizeof(cfg));
  cfg.gridDim = dim3(grid, 1, 1);
  cfg.blockDim = dim3(MODE == MODE_GATHER ? GATHER_THREADS : GEMM_THREADS, 1, 1);
  cfg.dynamicSmemBytes = Cfg::SMEM_BYTES;
  cfg.stream = stream;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeClusterDimension;
  attr[0].val.clusterDim.x = CG;
  attr[0].val.clusterDim.y = 1;
  attr[0].val.clusterDim.z = 1;
  cfg.attrs = attr;
  cfg.numAttrs = 1;
  cudaError_t e = cudaLaunchKernelEx(&cfg, gemm_bf16_tcgen05_kernel<BLOCK_N, CG, MODE>, maps, *mc, args, fa);
  if (e != cudaSuccess) return -(int)e;
  return -(int)cudaGetLastError();
}

template <int BLOCK_N, int CG, int MODE = MODE_PLAIN>
int launch_gemm(const void* A, const void* B, const GemmArgs& args, const FusedArgs& fa, long long lda, long long ldb, int sm_limit,
                cudaStream_t stream) {
  const Operands one = {A, B, lda, ldb, args.M, args.N};
  return launch_gemm<BLOCK_N, CG, MODE>(&one, 1, args, fa, sm_limit, stream);
}

// Tile shape for a problem: CTA pairs (256 x 256 tiles, half of B per CTA) whenever both extents fill such a tile; single
// CTAs with 128 x 256 or 128 x 128 tiles for small or ragged problems.
int dispatch_gemm(const void* A, const void* B, const GemmArgs& args, const FusedArgs& fa, long long lda, long long ldb, int sm_limit,
                  cudaStream_t s) {
  const int M = args.M, N = args.N;
  const bool use256 = (N >= 256) && ((N % 256 == 0) || (N % 256 > 128) || N >= 2048);
  static const int force_cg = [] {
    const char* v = getenv("YAFSDP_GEMM_CTA_GROUP");
    return v ? atoi(v) : 0;
  }();
  const bool pair_ok = use256 && M >= 256 && (M % 256 == 0 || M % 256 > 128 || M >= 2048);
  if (fa.gather) {
    if (pair_ok && force_cg != 1) return launch_gemm<256, 2, MODE_GATHER>(A, B, args, fa, lda, ldb, sm_limit, s);
    return use256 ? launch_gemm<256, 1, MODE_GATHER>(A, B, args, fa, lda, ldb, sm_limit, s)
                  : launch_gemm<128, 1, MODE_GATHER>(A, B, args, fa, lda, ldb, sm_limit, s);
  }
  if (fa.scatter) {
    if (pair_ok && force_cg != 1) return launch_gemm<256, 2, MODE_SCATTER>(A, B, args, fa, lda, ldb, sm_limit, s);
    return use256 ? launch_gemm<256, 1, MODE_SCATTER>(A, B, args, fa, lda, ldb, sm_limit, s)
                  : launch_gemm<128, 1, MODE_SCATTER>(A, B, args, fa, lda, ldb, sm_limit, s);
  }
  if (pair_ok && force_cg != 1) return launch_gemm<256, 2>(A, B, args, fa, lda, ldb, sm_limit, s);
  return use256 ? launch_gemm<256, 1>(A, B, args, fa, lda, ldb, sm_limit, s) : launch_gemm<128, 1>(A, B, args, fa, lda, ldb, sm_limit, s);
}

}  // namespace

// C[M,N] = alpha * A * B^T (+ C).  A is [M,K] with row pitch lda (a_mn = 0) or stored as [K,M] with row
// pitch lda (a_mn = 1); B likewise as [N,K] (b_mn = 0) or [K,N] (b_mn = 1).  bf16 inputs; C is bf16 or
// fp32 (out_f32) with row pitch ldc.  Pitches are in elements and must be multiples of 8 (16-byte TMA
// strides); base pointers must be 16-byte aligned.  sm_limit > 0 caps the persistent grid (leaves SMs
// to a concurrent communication kernel).
extern "C" int yf_gemm_bf16_sumsq(const void* A, const void* B, void* C, int M, int N, int K, long long lda, long long ldb,
                                  long long ldc, int a_mn, int b_mn, int out_f32, int accumulate, float alpha, int sm_limit,
                                  float* sumsq, void* stream);

extern "C" int yf_gemm_bf16(const void* A, const void* B, void* C, int M, int N, int K, long long lda, long long ldb,
                            long long ldc, int a_mn, int b_mn, int out_f32, int accumulate, float alpha, int sm_limit,
                            void* stream) {
  return yf_gemm_bf16_sumsq(A, B, C, M, N, K, lda, ldb, ldc, a_mn, b_mn, out_f32, accumulate, alpha, sm_limit, nullptr, stream);
}

// Same as yf_gemm_bf16; when `sumsq` is given (fp32 output, no accumulation) the kernel also adds the sum of squares
// of everything it wrote to *sumsq, so a gradient norm needs no extra pass over a freshly written weight gradient.
extern "C" int yf_gemm_bf16_sumsq(const void* A, const void* B, void* C, int M, int N, int K, long long lda, long long ldb,
                                  long long ldc, int a_mn, int b_mn, int out_f32, int accumulate, float alpha, int sm_limit,
                                  float* sumsq, void* stream) {
  if (M <= 0 || N <= 0 || K <= 0) return -1;
  if (sumsq != nullptr && (!out_f32 || accumulate)) return -1;
  if ((lda % 8) || (ldb % 8) || (ldc % (out_f32 ? 4 : 8))) return -1;
  if ((reinterpret_cast<uintptr_t>(A) | reinterpret_cast<uintptr_t>(B) | reinterpret_cast<uintptr_t>(C)) & 15) return -1;
  GemmArgs args;
  memset(&args, 0, sizeof(args));
  args.C = C;
  args.M = M; args.N = N; args.K = K;
  args.ldc = ldc;
  args.alpha = alpha;
  args.a_mn = a_mn ? 1 : 0;
  args.b_mn = b_mn ? 1 : 0;
  args.out_f32 = out_f32 ? 1 : 0;
  args.accumulate = accumulate ? 1 : 0;
  cudaStream_t s = reinterpret_cast<cudaStream_t>(stream);
  // 128x256 tiles unless N is small or the 256-wide tiling wastes more of the last column block
  FusedArgs fa;
  memset(&fa, 0, sizeof(fa));
  fa.sumsq = sumsq;
  return dispatch_gemm(A, B, args, fa, lda, ldb, sm_limit, s);
}

// C[M,N] = alpha * A * B^T + R with a bf16 residual R [M,N] (row pitch ldr) added in fp32 before the bf16 output is rounded;
// C may be R itself.  N, ldr multiples of 8; R 16-byte aligned.
extern "C" int yf_gemm_bf16_residual(const void* A, const void* B, void* C, const void* R, int M, int N, int K, long long lda,
                                     long long ldb, long long ldc, long long ldr, int a_mn, int b_mn, float alpha, int sm_limit,
                                     void* stream) {
  if (M <= 0 || N <= 0 || K <= 0 || R == nullptr) return -1;
  if ((lda % 8) || (ldb % 8) || (ldc % 8) || (ldr % 8) || (N % 8) || (reinterpret_cast<uintptr_t>(R) & 15)) return -1;
  GemmArgs args;
  memset(&args, 0, sizeof(args));
  args.C = C;
  args.M = M; args.N = N; args.K = K;
  args.ldc = ldc;
  args.alpha = alpha;
  args.a_mn = a_mn ? 1 : 0;
  args.b_mn = b_mn ? 1 : 0;
  args.R = R;
  args.ldr = ldr;
  FusedArgs fa;
  memset(&fa, 0, sizeof(fa));
  return dispatch_gemm(A, B, args, fa, lda, ldb, sm_limit, reinterpret_cast<cudaStream_t>(stream));
}

// All-gather -> GEMM in one kernel.  C[M,N] = A[M,K] * B[N,K]^T where B (row-major, contiguous, K-major) is a
// sub-range of the layer's flat bf16 parameter buffer that the same kernel gathers:
//   peer_in[r]  : rank r's shard (shard_bytes bytes) of the layer, peer-mapped; entry `rank` is the local shard
//   layer_buf   : local unsharded layer buffer (world * shard_bytes bytes); B = layer_buf + b_byte_off
//   counters    : one unsigned 64-bit word per B column block of 256 rows (128 when N < 256), in this GPU's memory, zero
//                 before the first call; epoch = 1, 2, ... counts the calls made with these counters and this shape
// On return (stream order) the whole layer buffer is filled, not only B.
extern "C" int yf_gemm_bf16_gathered(const void* A, void* C, int M, int N, int K, long long lda, long long ldc, int a_mn,
                                     int out_f32, void* const* peer_in, void* layer_buf, long long shard_bytes,
                                     long long b_byte_off, int rank, int world, void* counters, long long epoch, void* stream) {
  if (M <= 0 || N <= 0 || K <= 0 || world < 1 || world > MAX_RANKS || rank < 0 || rank >= world) return -1;
  if ((lda % 8) || (K % 8) || (ldc % (out_f32 ? 4 : 8)) || epoch <= 0 || counters == nullptr) return -1;
  if ((shard_bytes % 16) || shard_bytes <= 0 || (b_byte_off % 16)) return -1;
  if (b_byte_off < 0 || b_byte_off + (long long)N * K * 2 > shard_bytes * world) return -1;
  const uint8_t* B = reinterpret_cast<const uint8_t*>(layer_buf) + b_byte_off;
  if ((reinterpret_cast<uintptr_t>(A) | reinterpret_cast<uintptr_t>(B) | reinterpret_cast<uintptr_t>(C) |
       reinterpret_cast<uintptr_t>(layer_buf)) & 15)
    return -1;
  GemmArgs args;
  memset(&args, 0, sizeof(args));
  args.C = C;
  args.M = M; args.N = N; args.K = K;
  args.ldc = ldc;
  args.alpha = 1.f;
  args.a_mn = a_mn ? 1 : 0;
  args.b_mn = 0;
  args.out_f32 = out_f32 ? 1 : 0;
  args.accumulate = 0;
  FusedArgs fa;
  memset(&fa, 0, sizeof(fa));
  fa.gather = 1;
  fa.world = world; fa.rank = rank;
  fa.counters = reinterpret_cast<unsigned long long*>(counters);
  fa.epoch = (unsigned long long)epoch;
  for (int r = 0; r < world; ++r) {
    if (!peer_in[r] || (reinterpret_cast<uintptr_t>(peer_in[r]) & 15)) return -1;
    fa.peer_in[r] = peer_in[r];
  }
  fa.layer_buf = reinterpret_cast<uint8_t*>(layer_buf);
  fa.shard_bytes = shard_bytes;
  fa.b_byte_off = b_byte_off;
  cudaStream_t s = reinterpret_cast<cudaStream_t>(stream);
  return dispatch_gemm(A, B, args, fa, lda, K, 0, s);
}

// GEMM -> reduce-scatter in one kernel.  dW[M,N] = A * B^T in fp32 is not stored locally: each 16-byte piece is
// pushed into the staging slot `rank` of the rank that owns its position c_flat_off + m*N + n of the flat layer
// gradient (peer_grad[o] = base of owner o's reduce buffer, laid out as `world` slots of shard_numel floats).
// wire_bf16: the slots hold bf16 instead of fp32 (half the NVLink bytes; the owner still sums in fp32).  shard_numel, N and
// c_flat_off must be multiples of 4 (8 with the bf16 wire).  The owners sum their slots afterwards
// (yf_reduce_scatter_pull on local slot pointers) once every rank's pushes are complete.
extern "C" int yf_gemm_bf16_scatter(const void* A, const void* B, int M, int N, int K, long long lda, long long ldb, int a_mn,
                                    int b_mn, float alpha, void* const* peer_grad, long long c_flat_off, long long shard_numel,
                                    int rank, int world, int wire_bf16, int sm_limit, void* stream) {
  if (M <= 0 || N <= 0 || K <= 0 || world < 1 || world > MAX_RANKS || rank < 0 || rank >= world) return -1;
  const int al = wire_bf16 ? 8 : 4;  // elements per 16 bytes on the wire
  if ((lda % 8) || (ldb % 8) || (N % al) || (shard_numel % al) || (c_flat_off % al) || c_flat_off < 0) return -1;
  if (c_flat_off + (long long)M * N > shard_numel * world) return -1;
  if ((reinterpret_cast<uintptr_t>(A) | reinterpret_cast<uintptr_t>(B)) & 15) return -1;
  GemmArgs args;
  memset(&args, 0, sizeof(args));
  args.C = peer_grad[rank];  // only used to build a (unused) store descriptor
  args.M = M; args.N = N; args.K = K;
  args.ldc = N;
  args.alpha = alpha;
  args.a_mn = a_mn ? 1 : 0;
  args.b_mn = b_mn ? 1 : 0;
  args.out_f32 = 1;
  args.accumulate = 0;
  FusedArgs fa;
  memset(&fa, 0, sizeof(fa));
  fa.scatter = 1;
  fa.wire_bf16 = wire_bf16 ? 1 : 0;
  fa.world = world; fa.rank = rank;
  for (int r = 0; r < world; ++r) {
    if (!peer_grad[r] || (reinterpret_cast<uintptr_t>(peer_grad[r]) & 15)) return -1;
    fa.peer_grad[r] = peer_grad[r];
  }
  fa.c_flat_off = c_flat_off;
  fa.shard_numel = shard_numel;
  cudaStream_t s = reinterpret_cast<cudaStream_t>(stream);
  return dispatch_gemm(A, B, args, fa, lda, ldb, sm_limit, s);
}

// The weight-gradient GEMMs of a whole layer as ONE launch, pushed to their owners (grouped GEMM -> reduce-scatter).
// n problems (at most 4) dW_i[M_i, N_i] = A_i^T-or-not * B_i, sharing K and the operand majors, in the order of their
// positions flat_off[i] in the flat layer gradient.  Every rank deals the owners' tiles round-robin (owner rank + 1 first), so
// it pushes to all owners all the time and no owner's NVLink ingress becomes a hot spot, which separate launches cannot
// avoid (all ranks would push the same rows, i.e. to the same one or two owners, at the same time).
extern "C" int yf_gemm_bf16_scatter_grouped(int n, const void* const* A, const void* const* B, const int* M, const int* N, int K,
                                            const long long* lda, const long long* ldb, int a_mn, int b_mn, float alpha,
                                            void* const* peer_grad, const long long* flat_off, long long shard_numel, int rank,
                                            int world, int wire_bf16, int sm_limit, void* stream) {
  const int al = wire_bf16 ? 8 : 4;  // elements per 16 bytes on the wire
  if (n < 1 || n > MAX_GROUP || K <= 0 || world < 1 || world > MAX_RANKS || rank < 0 || rank >= world || (shard_numel % al)) return -1;
  GemmArgs args;
  memset(&args, 0, sizeof(args));
  Operands ops[MAX_GROUP];
  bool all256 = true;
  for (int i = 0; i < n; ++i) {
    if (M[i] <= 0 || N[i] <= 0 || (lda[i] % 8) || (ldb[i] % 8) || (N[i] % al) || (flat_off[i] % al) || flat_off[i] < 0) return -1;
    if (flat_off[i] + (long long)M[i] * N[i] > shard_numel * world) return -1;
    if (i > 0 && flat_off[i] < flat_off[i - 1] + (long long)M[i - 1] * N[i - 1]) return -1;  // ascending, no overlap
    if ((reinterpret_cast<uintptr_t>(A[i]) | reinterpret_cast<uintptr_t>(B[i])) & 15) return -1;
    ops[i] = {A[i], B[i], lda[i], ldb[i], M[i], N[i]};
    args.Mp[i] = M[i];
    args.Np[i] = N[i];
    args.flat_off[i] = flat_off[i];
    all256 = all256 && M[i] >= 256 && N[i] >= 256;
  }
  args.n_prob = n;
  args.C = peer_grad[rank];  // only used to build a (unused) store descriptor
  args.M = M[0]; args.N = N[0]; args.K = K;
  args.ldc = N[0];
  args.alpha = alpha;
  args.a_mn = a_mn ? 1 : 0;
  args.b_mn = b_mn ? 1 : 0;
  args.out_f32 = 1;
  FusedArgs fa;
  memset(&fa, 0, sizeof(fa));
  fa.scatter = 1;
  fa.wire_bf16 = wire_bf16 ? 1 : 0;
  fa.world = world; fa.rank = rank;
  for (int r = 0; r < world; ++r) {
    if (!peer_grad[r] || (reinterpret_cast<uintptr_t>(peer_grad[r]) & 15)) return -1;
    fa.peer_grad[r] = peer_grad[r];
  }
  fa.shard_numel = shard_numel;
  cudaStream_t s = reinterpret_cast<cudaStream_t>(stream);
  if (all256) return launch_gemm<256, 2, MODE_SCATTER>(ops, n, args, fa, sm_limit, s);
  return launch_gemm<128, 1, MODE_SCATTER>(ops, n, args, fa, sm_limit, s);
}
