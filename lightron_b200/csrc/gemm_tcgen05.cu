// bf16 GEMM for sm_100a:  C[M,N] = op(A) * op(B)^T with fp32 accumulation in tensor memory.
//
//   * operands are staged in shared memory by TMA (cp.async.bulk.tensor, 128-byte swizzle,
//     no cluster multicast) through a 4-stage mbarrier ring;
//   * one elected thread issues tcgen05.mma (cta_group::1, kind::f16, 128x256x16 per
//     instruction) with shared-memory matrix descriptors;
//   * accumulators live in TMEM: 2 buffers x 256 columns, so the epilogue of tile i (tcgen05.ld ->
//     bf16 -> global) overlaps the main loop of tile i+1;
//   * persistent: one CTA per SM walks the tile list in an L2-friendly grouped order;
//   * both operand majors are supported so that forward (x W^T), dgrad (dy W) and wgrad
//     (dy^T x) all read the tensors as they sit in memory, with no transposes:
//        a_mn = 0: A stored [M, K] (K contiguous)      a_mn = 1: A stored [K, M] (M contiguous)
//        b_mn = 0: B stored [N, K] (K contiguous)      b_mn = 1: B stored [K, N] (N contiguous)
//   * every mbarrier wait is bounded; on expiry the kernel records a status code, stops issuing
//     work, frees its TMEM and returns.
//
// Warp roles (192 threads): warp 0 = TMA producer, warp 1 = TMEM allocator + MMA issuer,
// warps 2..5 = epilogue (warp w reads TMEM lanes 32*(w%4) .. +31).
#include <cuda.h>
#include <string.h>
#include "common.cuh"
#include "tcgen05.cuh"
#include "comm.cuh"

// Device-side status words of the GEMM kernels.  A bounded wait that runs out sets word 0 to a
// non-zero code and word 1 to a location id instead of spinning forever; the host reads them
// with lb_device_status().
static __device__ unsigned int g_lb_dev_status[4] = {0, 0, 0, 0};

namespace {

constexpr int BM = 128, BN = 256, BK = 64;
constexpr int STAGES = 4;
constexpr int STAGES_DEFAULT = STAGES;
constexpr int A_BYTES = BM * BK * 2;  // 16 KiB
constexpr int B_BYTES = BN * BK * 2;  // 32 KiB
constexpr int STAGE_BYTES = A_BYTES + B_BYTES;
constexpr int SMEM_BYTES = STAGES * STAGE_BYTES + 1024 /*alignment slack*/ + 256 /*barriers*/;
constexpr int NUM_THREADS = 192;
constexpr int GROUP_M = 8;

// The PTX wrappers (mbarrier, TMA, tcgen05, descriptors, tensor maps) live in tcgen05.cuh, the
// flag primitives in comm.cuh.
using namespace bw;

// Bounded mbarrier wait that also records where it gave up.
__device__ __forceinline__ bool mbar_wait(uint32_t bar, uint32_t parity, volatile int* abort_flag, unsigned where) {
  if (bw::mbar_wait(bar, parity, abort_flag)) return true;
  if (atomicCAS(&g_lb_dev_status[0], 0u, 1u) == 0u) atomicExch(&g_lb_dev_status[1], where);
  return false;
}
__device__ __forceinline__ void tcgen05_fence_before() { fence_before(); }
__device__ __forceinline__ void tcgen05_fence_after() { fence_after(); }

struct GemmParams {
  int M, N, K;
  long long ldc;
  int a_mn, b_mn;
  int tiles_m, tiles_n, num_tiles, num_kb;
};

// Extra arguments of the fused compute + collective variants (tensor-parallel group of n ranks
// whose buffers are mapped into every rank's address space; all pointers below are usable from
// this GPU, peers' ones go over NVLink).
//   MODE 1, all-gather -> GEMM:  A = gather_over_ranks(x_local)  [M, K], this rank owns rows
//     [rank * rows_per_rank, ...).  CTAs 0 .. n_comm-1 PUSH this rank's rows into every rank's
//     gather buffer (coalesced 16-byte stores through peer pointers: stores are fire-and-forget,
//     so a few CTAs saturate NVLink, which latency-bound remote loads cannot) and count each
//     128-row block in the destination's flag word; the other CTAs run the tcgen05 main loop,
//     local rows first (read straight from x_local), each remote tile gated on its flag.
//   MODE 2, GEMM -> reduce-scatter:  every rank computes partial C = A_local B_local^T [M, N].
//     Tiles of rows that another rank keeps come first: the epilogue stages each in shared memory
//     and stores it, 512 contiguous bytes per row, straight into the owner's receive area and
//     counts it in the owner's flag word.  Tiles of the rows this rank keeps come last: their
//     epilogue waits (bounded) for the peers' partials of that row block, adds them to the
//     accumulator and stores the final bf16 rows, so the reduction costs no extra pass.
constexpr int MAX_RANKS = 8;
constexpr int MOVER_WARPS = NUM_THREADS / 32;
struct CommParams {
  int n_ranks, rank, rows_per_rank, blocks_per_rank;   // blocks of BM rows
  int n_comm;                                          // MODE 1: CTAs that move data
  unsigned int ag_target;                              // MODE 1: flag value when a block has fully arrived
  unsigned int rs_target;                              // MODE 2: counter value when a block is complete
  const bf16* x_local;                                 // MODE 1: this rank's rows [rows_per_rank, K], row stride ld_x
  long long ld_x;
  bf16* gather[MAX_RANKS];                             // MODE 1: rank r's gather buffer [M, K] contiguous
  unsigned int* ag_flags[MAX_RANKS];                   // MODE 1: rank r's block counters [M / 128]
  bf16* recv[MAX_RANKS];                               // MODE 2: rank r's receive area [n_ranks][rows_per_rank][N]
  unsigned int* rs_flags[MAX_RANKS];                   // MODE 2: rank r's counters [n_ranks][blocks_per_rank]
  bf16* out;                                           // MODE 2: reduced [rows_per_rank, N]
  long long ld_out;
  unsigned long long wait_ns;                          // limit of every wait on a peer's flag
};

__device__ __forceinline__ void tile_coords(int t, const GemmParams& p, int& tm, int& tn) {
  const int group_size = GROUP_M * p.tiles_n;
  const int group = t / group_size;
  const int first_m = group * GROUP_M;
  const int gsz = min(p.tiles_m - first_m, GROUP_M);
  const int in_group = t - group * group_size;
  tm = first_m + in_group % gsz;
  tn = in_group / gsz;
}

using lbcomm::red_release_sys_add;
// Bounded wait on a flag written by another CTA or another GPU; records the failure.
__device__ __forceinline__ bool flag_wait_ge(const unsigned int* f, unsigned int target, unsigned long long limit_ns, unsigned where) {
  if (lbcomm::flag_wait_ge(f, target, limit_ns)) return true;
  atomicExch(&g_lb_dev_status[0], 2u);
  atomicExch(&g_lb_dev_status[1], where);
  return false;
}

// MODE 2 stages its output tile in shared memory (one padded 32 x 256 bf16 panel per epilogue warp)
// and pays for it with one pipeline stage.
constexpr int RS_ROW_BYTES = BN * 2 + 16;                 // padded: 16-byte stores of a warp stay conflict-free
constexpr int RS_STAGE_BYTES = 4 * 32 * RS_ROW_BYTES;
constexpr int STAGES_RS = 3;
constexpr int SMEM_BYTES_RS = STAGES_RS * STAGE_BYTES + 1024 + 1024 + RS_STAGE_BYTES;
// One tile of the producer / of the MMA issuer with the operand majors as compile-time constants:
// descriptor fields and the number of TMA boxes become constants in the single-thread issue loops
// (measured 3-8 % faster than run-time majors).
template <int NSTAGES, bool A_MN, bool B_MN>
__device__ __forceinline__ bool produce_tile(const CUtensorMap* ta, const CUtensorMap* tb, int m0, int n0, int num_kb,
                                             uint32_t smem_base, uint32_t bar_base, int& stage, uint32_t& phase,
                                             volatile int* abort_flag) {
  for (int kb = 0; kb < num_kb; kb++) {
    if (!mbar_wait(bar_base + 8u * (NSTAGES + stage), phase ^ 1u, abort_flag, 1u)) return false;
    const uint32_t fb = bar_base + 8u * stage;
    mbar_expect_tx(fb, STAGE_BYTES);
    const uint32_t sa = smem_base + stage * STAGE_BYTES;
    const uint32_t sb = sa + A_BYTES;
    const int k0 = kb * BK;
    if (!A_MN) {
      tma_load_2d(sa, ta, k0, m0, fb);                                                      // box {64 k, 128 m}
    } else {
#pragma unroll
      for (int j = 0; j < BM / 64; j++) tma_load_2d(sa + j * 8192, ta, m0 + 64 * j, k0, fb);  // box {64 m, 64 k}
    }
    if (!B_MN) {
      tma_load_2d(sb, tb, k0, n0, fb);                                                      // box {64 k, 256 n}
    } else {
#pragma unroll
      for (int j = 0; j < BN / 64; j++) tma_load_2d(sb + j * 8192, tb, n0 + 64 * j, k0, fb);  // box {64 n, 64 k}
    }
    if (++stage == NSTAGES) { stage = 0; phase ^= 1u; }
  }
  return true;
}

template <int NSTAGES, bool A_MN, bool B_MN>
__device__ __forceinline__ bool mma_tile(uint32_t d_tmem, int num_kb, uint32_t smem_base, uint32_t bar_base, int& stage,
                                         uint32_t& phase, volatile int* abort_flag) {
  // instruction descriptor: D=f32, A=B=bf16, majors, N>>3 at bit 17, M>>4 at bit 24
  constexpr uint32_t idesc = (1u << 4) | (1u << 7) | (1u << 10) | ((A_MN ? 1u : 0u) << 15) | ((B_MN ? 1u : 0u) << 16) |
                             ((uint32_t)(BN >> 3) << 17) | ((uint32_t)(BM >> 4) << 24);
  constexpr uint32_t a_lbo = A_MN ? 8192u : 16u, b_lbo = B_MN ? 8192u : 16u;
  constexpr uint32_t a_kstep = A_MN ? 2048u : 32u, b_kstep = B_MN ? 2048u : 32u;   // bytes per K=16 slice
  for (int kb = 0; kb < num_kb; kb++) {
    if (!mbar_wait(bar_base + 8u * stage, phase, abort_flag, 3u)) return false;
    tcgen05_fence_after();
    const uint32_t sa = smem_base + stage * STAGE_BYTES;
    const uint32_t sb = sa + A_BYTES;
#pragma unroll
    for (int k = 0; k < BK / 16; k++) {
      const uint64_t ad = make_desc(sa + k * a_kstep, a_lbo, 1024u);
      const uint64_t bd = make_desc(sb + k * b_kstep, b_lbo, 1024u);
      umma_bf16(d_tmem, ad, bd, idesc, (kb | k) ? 1u : 0u);
    }
    umma_commit(bar_base + 8u * (NSTAGES + stage));  // frees this smem stage when the MMAs have read it
    if (++stage == NSTAGES) { stage = 0; phase ^= 1u; }
  }
  return true;
}

template <int MODE>
__global__ void __launch_bounds__(NUM_THREADS, 1)
gemm_bf16_kernel(const __grid_constant__ CUtensorMap tmap_a, const __grid_constant__ CUtensorMap tmap_b,
                 const __grid_constant__ CUtensorMap tmap_own, bf16* __restrict__ C, const GemmParams p,
                 const CommParams cp) {
  constexpr int STAGES = (MODE == 2) ? STAGES_RS : STAGES_DEFAULT;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~(uintptr_t)1023);
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + STAGES * STAGE_BYTES);
  // bars: [0,STAGES) full, [STAGES,2*STAGES) empty, then tmem_full[2], tmem_empty[2]
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 2 * STAGES + 4);
  __shared__ int s_abort[2];     // {abort, extra wait in ms}: see bw::mbar_wait

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;

  if (MODE == 1 && (int)blockIdx.x < cp.n_comm) {
    // ---------------- all-gather mover CTAs (no tensor-core work, no TMEM) ----------------
    // unit = (destination rank, 128-row block of this rank's rows).  Every warp copies its share of
    // the block's rows (two rows = 2 x K x 2 bytes in flight per warp), fences, and adds one to the
    // destination's counter of that block; warps never wait for each other, so while one sits in
    // its fence the others keep streaming.  Peers first, the local copy last.
    // (Measured alternatives on 2 GPUs, all slower inside this kernel although a plain copy kernel with
    // the same access pattern moves 630 GB/s with 16 CTAs: flat CTA-wide copies with one fence per block,
    // a signalling warp that fences while the others copy, and one fence per CTA after all its blocks.
    // A system-scope fence here does not return before the SM's queued peer stores have drained, so
    // what counts is that the warps of a CTA reach their fences at different times.)
    const int units = cp.n_ranks * cp.blocks_per_rank;
    const int vec_per_row = p.K / 8;
    for (int u = blockIdx.x; u < units; u += cp.n_comm) {
      const int dst_rank = (cp.rank + 1 + u / cp.blocks_per_rank) % cp.n_ranks;
      const int rb = u % cp.blocks_per_rank;
      const uint4* sp = reinterpret_cast<const uint4*>(cp.x_local + (size_t)rb * BM * cp.ld_x);
      uint4* dp = reinterpret_cast<uint4*>(cp.gather[dst_rank] + ((size_t)cp.rank * cp.rows_per_rank + (size_t)rb * BM) * p.K);
      const size_t src_row = (size_t)cp.ld_x / 8;
      // each warp owns rows warp, warp+6, ...; it keeps 4 rows x 4 vectors (256 B per lane) in flight
      for (int r = warp; r < BM; r += 4 * MOVER_WARPS) {
        for (int v0 = 0; v0 < vec_per_row; v0 += 32 * 4) {
          uint4 a[4][4];
#pragma unroll
          for (int q = 0; q < 4; q++) {
            const int rr = r + q * MOVER_WARPS;
#pragma unroll
            for (int j = 0; j < 4; j++) {
              const int v = v0 + j * 32 + lane;
              if (rr < BM && v < vec_per_row) a[q][j] = sp[(size_t)rr * src_row + v];
            }
          }
#pragma unroll
          for (int q = 0; q < 4; q++) {
            const int rr = r + q * MOVER_WARPS;
#pragma unroll
            for (int j = 0; j < 4; j++) {
              const int v = v0 + j * 32 + lane;
              if (rr < BM && v < vec_per_row) dp[(size_t)rr * vec_per_row + v] = a[q][j];
            }
          }
        }
      }
      __threadfence_system();
      __syncwarp();
      if (lane == 0) red_release_sys_add(cp.ag_flags[dst_rank] + cp.rank * cp.blocks_per_rank + rb, 1u);
    }
    return;
  }

  const uint32_t smem_base = smem_u32(smem);
  const uint32_t bar_base = smem_u32(bars);
  auto full_bar = [&](int s) { return bar_base + 8u * s; };
  auto empty_bar = [&](int s) { return bar_base + 8u * (STAGES + s); };
  auto tfull_bar = [&](int a) { return bar_base + 8u * (2 * STAGES + a); };
  auto tempty_bar = [&](int a) { return bar_base + 8u * (2 * STAGES + 2 + a); };
  // persistent tile walk of this CTA
  const int cta = (MODE == 1) ? (int)blockIdx.x - cp.n_comm : (int)blockIdx.x;
  const int n_cta = (MODE == 1) ? (int)gridDim.x - cp.n_comm : (int)gridDim.x;
  // m-block rotation: MODE 1 starts with the rows this rank already has, MODE 2 ends with the
  // rows this rank keeps (so that tiles that must travel are produced first)
  const int m_rot = (MODE == 1) ? cp.rank * cp.blocks_per_rank
                                : (MODE == 2 ? ((cp.rank + 1) % cp.n_ranks) * cp.blocks_per_rank : 0);
  auto map_tile = [&](int t, int& tm, int& tn) {
    tile_coords(t, p, tm, tn);
    if (MODE != 0) { tm += m_rot; if (tm >= p.tiles_m) tm -= p.tiles_m; }
  };

  if (threadIdx.x == 0) {
    s_abort[0] = 0;
    s_abort[1] = (MODE == 0) ? 0 : wait_extra_ms(cp.wait_ns);
    for (int s = 0; s < STAGES; s++) {
      mbar_init(full_bar(s), 1);
      mbar_init(empty_bar(s), 1);
    }
    for (int a = 0; a < 2; a++) {
      mbar_init(tfull_bar(a), 1);
      mbar_init(tempty_bar(a), 4);
    }
    mbar_init_fence();
    prefetch_tmap(&tmap_a);
    prefetch_tmap(&tmap_b);
  }
  if (warp == 1) {  // allocate all 512 TMEM columns (one CTA per SM by construction)
    tmem_alloc(smem_u32(tmem_slot), 512);
  }
  tcgen05_fence_before();
  __syncthreads();
  tcgen05_fence_after();
  const uint32_t tmem_base = *tmem_slot;
  volatile int* abort_flag = s_abort;

  if (warp == 0) {
    // ------------------------------ TMA producer ------------------------------
    if (lane == 0) {
      int stage = 0;
      uint32_t phase = 0;
      bool ok = true;
      for (int t = cta; t < p.num_tiles && ok; t += n_cta) {
        int tm, tn;
        map_tile(t, tm, tn);
        const int m0 = tm * BM, n0 = tn * BN;
        bool own = false;
        if (MODE == 1) {
          own = (tm / cp.blocks_per_rank) == cp.rank;
          if (!own) {
            // rows of this tile must have landed in this rank's gather buffer (pushed by a peer):
            // acquire the flag, then order those writes before the async-proxy reads
            if (!flag_wait_ge(cp.ag_flags[cp.rank] + tm, cp.ag_target, cp.wait_ns, 11u)) { *abort_flag = 1; ok = false; break; }
            asm volatile("fence.proxy.async;" ::: "memory");
          }
        }
        const int m0_own = m0 - cp.rank * cp.rows_per_rank;   // row inside this rank's own buffer
        const CUtensorMap* ta = (MODE == 1 && own) ? &tmap_own : &tmap_a;   // this rank's rows need no gather
        const int ma = (MODE == 1 && own) ? m0_own : m0;
        switch (p.a_mn * 2 + p.b_mn) {
          case 0: ok = produce_tile<STAGES, false, false>(ta, &tmap_b, ma, n0, p.num_kb, smem_base, bar_base, stage, phase, abort_flag); break;
          case 1: ok = produce_tile<STAGES, false, true>(ta, &tmap_b, ma, n0, p.num_kb, smem_base, bar_base, stage, phase, abort_flag); break;
          case 2: ok = produce_tile<STAGES, true, false>(ta, &tmap_b, ma, n0, p.num_kb, smem_base, bar_base, stage, phase, abort_flag); break;
          default: ok = produce_tile<STAGES, true, true>(ta, &tmap_b, ma, n0, p.num_kb, smem_base, bar_base, stage, phase, abort_flag); break;
        }
      }
    }
  } else if (warp == 1) {
    // ------------------------------ MMA issuer ------------------------------
    if (lane == 0) {
      int stage = 0;
      uint32_t phase = 0;
      bool ok = true;
      int it = 0;
      for (int t = cta; t < p.num_tiles && ok; t += n_cta, it++) {
        const int acc = it & 1;
        const uint32_t acc_phase = (uint32_t)(it >> 1) & 1u;
        if (!mbar_wait(tempty_bar(acc), acc_phase ^ 1u, abort_flag, 2u)) { ok = false; break; }
        tcgen05_fence_after();
        const uint32_t d_tmem = tmem_base + (uint32_t)acc * BN;
        switch (p.a_mn * 2 + p.b_mn) {
          case 0: ok = mma_tile<STAGES, false, false>(d_tmem, p.num_kb, smem_base, bar_base, stage, phase, abort_flag); break;
          case 1: ok = mma_tile<STAGES, false, true>(d_tmem, p.num_kb, smem_base, bar_base, stage, phase, abort_flag); break;
          case 2: ok = mma_tile<STAGES, true, false>(d_tmem, p.num_kb, smem_base, bar_base, stage, phase, abort_flag); break;
          default: ok = mma_tile<STAGES, true, true>(d_tmem, p.num_kb, smem_base, bar_base, stage, phase, abort_flag); break;
        }
        if (ok) umma_commit(tfull_bar(acc));  // accumulator complete
      }
    }
  } else {
    // ------------------------------ epilogue (4 warps) ------------------------------
    const int quad = warp & 3;  // TMEM lane quadrant this warp may access
    bool ok = true;
    int it = 0;
    constexpr int RS_MAX_PEND = 24;
    unsigned int* rs_pend[RS_MAX_PEND];     // MODE 2: counters of tiles whose stores are not yet fenced
    int rs_npend = 0, rs_pend_owner = -1;
    for (int t = cta; t < p.num_tiles && ok; t += n_cta, it++) {
      const int acc = it & 1;
      const uint32_t acc_phase = (uint32_t)(it >> 1) & 1u;
      int tm, tn;
      map_tile(t, tm, tn);
      if (!mbar_wait(tfull_bar(acc), acc_phase, abort_flag, 4u)) { ok = false; break; }
      tcgen05_fence_after();
      const int row = tm * BM + quad * 32 + lane;
      const int n0 = tn * BN;
      const uint32_t taddr = tmem_base + ((uint32_t)(quad * 32) << 16) + (uint32_t)acc * BN;
      bf16* crow;
      int owner = 0, lb = 0;
      if (MODE == 2) {
        // destination: receive area of the rank that owns this row block, slot of this rank
        owner = tm / cp.blocks_per_rank;
        lb = tm - owner * cp.blocks_per_rank;
        crow = cp.recv[owner] + ((size_t)cp.rank * cp.rows_per_rank + (size_t)lb * BM + quad * 32 + lane) * p.N + n0;
      } else {
        crow = C + (size_t)row * p.ldc + n0;
      }
      if (MODE == 2 && owner == cp.rank) {
        // Rows that this rank keeps (its tiles come last in the tile order, so the peers' partials of
        // these rows, which they produce FIRST, are on their way or already in the receive area):
        // wait for them, add them to the accumulator and store the finished bf16 rows.  No trip
        // through the receive area for the own partial, no second kernel for the sum.  (Parking the
        // tiles whose partials are not in yet and summing them after the main loop was measured
        // slower: the wait only moves to the end of the kernel, and the sum is then serial.)
        if (rs_npend > 0) {
          // the counts of the tiles already sent must leave before this rank starts waiting for its
          // peers: they are waiting for exactly those counts
          __threadfence_system();
          __syncwarp();
          if (lane == 0)
            for (int i = 0; i < rs_npend; i++) red_release_sys_add(rs_pend[i], 1u);
          rs_npend = 0;
        }
        bool arrived = true;
        for (int s = 0; s < cp.n_ranks; s++)
          if (s != cp.rank && !flag_wait_ge(cp.rs_flags[cp.rank] + s * cp.blocks_per_rank + lb, cp.rs_target, cp.wait_ns, 21u))
            arrived = false;
        const size_t lrow = (size_t)lb * BM + quad * 32 + lane;           // row inside this rank's [rows_per_rank, N]
        bf16* orow = cp.out + lrow * cp.ld_out + n0;
        // The partials of a 32-column chunk are loaded together (a store between two loads would
        // order the second load behind it).
        auto peer_row = [&](int s) { return cp.recv[cp.rank] + ((size_t)s * cp.rows_per_rank + lrow) * p.N + n0; };
        auto fetch = [&](uint4* q, int s, int c) {
          const bf16* src = peer_row(s) + c * 32;
#pragma unroll
          for (int g = 0; g < 4; g++)
            q[g] = (arrived && n0 + c * 32 + g * 8 < p.N) ? __ldcg(reinterpret_cast<const uint4*>(src + g * 8)) : make_uint4(0, 0, 0, 0);
        };
        auto add_store = [&](float* f, int c) {
#pragma unroll
          for (int g = 0; g < 4; g++)
            if (arrived && n0 + c * 32 + g * 8 < p.N) *reinterpret_cast<uint4*>(orow + c * 32 + g * 8) = pack8(f + g * 8);
        };
        if (cp.n_ranks == 2) {
          // one peer: its chunk c + 1 is in flight while chunk c is summed and stored
          const int s = cp.rank ^ 1;
          uint4 pq[2][4];
          fetch(pq[0], s, 0);
#pragma unroll
          for (int c = 0; c < BN / 32; c++) {
            if (c + 1 < BN / 32) fetch(pq[(c + 1) & 1], s, c + 1);
            uint32_t r[32];
            tmem_ld32(taddr + c * 32, r);
            tmem_ld_wait();
            float f[32];
#pragma unroll
            for (int g = 0; g < 4; g++) {
              float o[8];
              unpack8(pq[c & 1][g], o);
#pragma unroll
              for (int i = 0; i < 8; i++) f[g * 8 + i] = __uint_as_float(r[g * 8 + i]) + o[i];
            }
            add_store(f, c);
          }
        } else {
#pragma unroll 1
          for (int c = 0; c < BN / 32; c++) {
            uint32_t r[32];
            tmem_ld32(taddr + c * 32, r);
            tmem_ld_wait();
            float f[32];
#pragma unroll
            for (int i = 0; i < 32; i++) f[i] = __uint_as_float(r[i]);
            for (int s = 0; s < cp.n_ranks; s++) {
              if (s == cp.rank) continue;
              uint4 pq[4];
              fetch(pq, s, c);
#pragma unroll
              for (int g = 0; g < 4; g++) {
                float o[8];
                unpack8(pq[g], o);
#pragma unroll
                for (int i = 0; i < 8; i++) f[g * 8 + i] += o[i];
              }
            }
            add_store(f, c);
          }
        }
        tcgen05_fence_before();
        __syncwarp();
        if (lane == 0) mbar_arrive(tempty_bar(acc));
        continue;
      }
      if (MODE == 2) {
        // TMEM -> registers -> padded smem panel of this warp -> one bulk store per row (512 B) to
        // the owner's receive area: NVLink sees large writes instead of scattered 16-byte stores.
        uint8_t* panel = smem + STAGES * STAGE_BYTES + 1024 + (warp - 2) * (32 * RS_ROW_BYTES);
        uint8_t* prow = panel + lane * RS_ROW_BYTES;
#pragma unroll 1
        for (int c = 0; c < BN / 32; c++) {
          uint32_t r[32];
          tmem_ld32(taddr + c * 32, r);
          tmem_ld_wait();
#pragma unroll
          for (int g = 0; g < 4; g++) {
            float f[8];
#pragma unroll
            for (int i = 0; i < 8; i++) f[i] = __uint_as_float(r[g * 8 + i]);
            *reinterpret_cast<uint4*>(prow + c * 64 + g * 16) = pack8(f);
          }
        }
        tcgen05_fence_before();
        __syncwarp();
        if (lane == 0) mbar_arrive(tempty_bar(acc));       // accumulator free: the next tile may start
        // Counting a tile needs a system-scope fence after its stores, and on NVLink that fence does
        // not return before everything this SM has stored to the peer has drained (tens of
        // microseconds).  The tiles that travel come first in the tile order, so their counts are
        // kept and sent together: one fence when the destination rank changes (tiles are ordered by
        // destination, so with two ranks that is when this CTA turns to the rows it keeps), when the
        // CTA ends, or when the list is full.
        if (rs_npend > 0 && (owner != rs_pend_owner || rs_npend == RS_MAX_PEND)) {
          __threadfence_system();
          __syncwarp();
          if (lane == 0)
            for (int i = 0; i < rs_npend; i++) red_release_sys_add(rs_pend[i], 1u);
          rs_npend = 0;
        }
        rs_pend_owner = owner;
        rs_pend[rs_npend++] = cp.rs_flags[owner] + cp.rank * cp.blocks_per_rank + lb;
        const int nvec = min(BN, p.N - n0) / 8;            // 16-byte vectors per row (<= 32)
        bf16* dst0 = cp.recv[owner] + ((size_t)cp.rank * cp.rows_per_rank + (size_t)lb * BM + quad * 32) * p.N + n0;
        if (lane < nvec) {
#pragma unroll 8
          for (int r = 0; r < 32; r++)                     // one 512-byte row per warp instruction
            *reinterpret_cast<uint4*>(dst0 + (size_t)r * p.N + lane * 8) =
                *reinterpret_cast<const uint4*>(panel + r * RS_ROW_BYTES + lane * 16);
        }
        __syncwarp();                                      // panel fully read before the next tile rewrites it
        continue;
      }
#pragma unroll 1
      for (int c = 0; c < BN / 32; c++) {
        uint32_t r[32];
        tmem_ld32(taddr + c * 32, r);
        tmem_ld_wait();
        if (row < p.M) {
#pragma unroll
          for (int g = 0; g < 4; g++) {
            const int col = n0 + c * 32 + g * 8;
            if (col < p.N) {  // N is a multiple of 8
              float f[8];
#pragma unroll
              for (int i = 0; i < 8; i++) f[i] = __uint_as_float(r[g * 8 + i]);
              *reinterpret_cast<uint4*>(crow + c * 32 + g * 8) = pack8(f);
            }
          }
        }
      }
      tcgen05_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(tempty_bar(acc));
    }
    if (MODE == 2 && rs_npend > 0) {
      __threadfence_system();
      __syncwarp();
      if (lane == 0)
        for (int i = 0; i < rs_npend; i++) red_release_sys_add(rs_pend[i], 1u);
    }
  }

  // ------------------------------ teardown ------------------------------
  tcgen05_fence_before();
  __syncthreads();
  if (warp == 1) {
    tcgen05_fence_after();
    tmem_dealloc(tmem_base, 512);
  }

}

// ---- host side --------------------------------------------------------------------------------
// 2-D bf16 tensor map: `inner` contiguous elements, `outer` rows of `ld` elements.
int make_map(CUtensorMap* m, const void* base, uint64_t inner, uint64_t outer, uint64_t ld, uint32_t box_inner,
             uint32_t box_outer) {
  return bw::make_map_bf16(m, base, inner, outer, ld, box_inner, box_outer);
}

int g_num_sms = 0;

}  // namespace

// Copies the 4 status words to host memory `out` (synchronous) and clears them.
extern "C" int lb_device_status(void* out) {
  cudaError_t e = cudaMemcpyFromSymbol(out, g_lb_dev_status, sizeof(unsigned int) * 4);
  if (e != cudaSuccess) { g_lb_last_cuda_error = (int)e; return LB_ERR_LAUNCH; }
  unsigned int zeros[4] = {0, 0, 0, 0};
  cudaMemcpyToSymbol(g_lb_dev_status, zeros, sizeof(zeros));
  return LB_OK;
}

// C[M,N] (row stride ldc) = op(A) op(B)^T, bf16 in / bf16 out, fp32 accumulate.
// Requirements: A, B, C 16-byte aligned; lda, ldb, ldc, N multiples of 8 elements.
extern "C" int lb_gemm_grouped(int n, const void* const* A, const void* const* B, void* const* C, const int* M,
                               const int* N, const int* K, const long long* lda, const long long* ldb,
                               const long long* ldc, const int* a_mn, const int* b_mn, const int* accumulate,
                               void* stream);

// flags bit 0: run the kernel of this file (majors as run-time values) instead of the grouped
// kernel with one problem, whose issue loops are specialised on the majors and measure 3-8 % faster.
extern "C" int lb_gemm_bf16(const void* A, const void* B, void* C, int M, int N, int K, long long lda, long long ldb,
                            long long ldc, int a_mn, int b_mn, int flags, void* stream) {
  if (!(flags & 1)) {
    const int acc = 0;
    return lb_gemm_grouped(1, &A, &B, &C, &M, &N, &K, &lda, &ldb, &ldc, &a_mn, &b_mn, &acc, stream);
  }
  if (M <= 0 || N <= 0 || K <= 0) return LB_ERR_SHAPE;
  if ((lda % 8) || (ldb % 8) || (ldc % 8) || (N % 8)) return LB_ERR_SHAPE;
  if (((uintptr_t)A | (uintptr_t)B | (uintptr_t)C) & 15) return LB_ERR_ARG;
  if (a_mn && (M % 8)) return LB_ERR_SHAPE;
  // The driver-API encode call needs a current context on THIS thread; autograd's backward
  // threads may not have touched the runtime yet.
  static thread_local bool ctx_bound = false;
  if (!ctx_bound) {
    cudaFree(0);
    ctx_bound = true;
  }
  CUtensorMap ta, tb;
  int rc;
  if (!a_mn) rc = make_map(&ta, A, (uint64_t)K, (uint64_t)M, (uint64_t)lda, BK, BM);
  else       rc = make_map(&ta, A, (uint64_t)M, (uint64_t)K, (uint64_t)lda, 64, BK);
  if (rc) return rc;
  if (!b_mn) rc = make_map(&tb, B, (uint64_t)K, (uint64_t)N, (uint64_t)ldb, BK, BN);
  else       rc = make_map(&tb, B, (uint64_t)N, (uint64_t)K, (uint64_t)ldb, 64, BK);
  if (rc) return rc;
  if (g_num_sms == 0) {
    int dev = 0;
    cudaGetDevice(&dev);
    cudaDeviceGetAttribute(&g_num_sms, cudaDevAttrMultiProcessorCount, dev);
    cudaFuncSetAttribute(gemm_bf16_kernel<0>, cudaFuncAttributeMaxDynamicSharedMemorySize, SMEM_BYTES);
    cudaFuncSetAttribute(gemm_bf16_kernel<1>, cudaFuncAttributeMaxDynamicSharedMemorySize, SMEM_BYTES);
    cudaFuncSetAttribute(gemm_bf16_kernel<2>, cudaFuncAttributeMaxDynamicSharedMemorySize, SMEM_BYTES_RS);
  }
  GemmParams p;
  p.M = M; p.N = N; p.K = K; p.ldc = ldc; p.a_mn = a_mn; p.b_mn = b_mn;
  p.tiles_m = (M + BM - 1) / BM;
  p.tiles_n = (N + BN - 1) / BN;
  p.num_tiles = p.tiles_m * p.tiles_n;
  p.num_kb = (K + BK - 1) / BK;
  int grid = p.num_tiles < g_num_sms ? p.num_tiles : g_num_sms;
  CommParams cp;
  memset(&cp, 0, sizeof(cp));
  gemm_bf16_kernel<0><<<grid, NUM_THREADS, SMEM_BYTES, (cudaStream_t)stream>>>(ta, tb, ta, (bf16*)C, p, cp);
  LB_CHECK_LAUNCH();
  return LB_OK;
}

namespace {
int init_sms() {
  if (g_num_sms == 0) {
    int dev = 0;
    cudaGetDevice(&dev);
    cudaDeviceGetAttribute(&g_num_sms, cudaDevAttrMultiProcessorCount, dev);
    cudaFuncSetAttribute(gemm_bf16_kernel<0>, cudaFuncAttributeMaxDynamicSharedMemorySize, SMEM_BYTES);
    cudaFuncSetAttribute(gemm_bf16_kernel<1>, cudaFuncAttributeMaxDynamicSharedMemorySize, SMEM_BYTES);
    cudaFuncSetAttribute(gemm_bf16_kernel<2>, cudaFuncAttributeMaxDynamicSharedMemorySize, SMEM_BYTES_RS);
  }
  return g_num_sms;
}
// raises `count` consecutive arrival counters by `inc` (after a copy-engine transfer has landed)
__global__ void ag_flag_bump_kernel(unsigned int* flags, int count, unsigned int inc) {
  for (int i = threadIdx.x; i < count; i += blockDim.x) {
    __threadfence_system();
    red_release_sys_add(flags + i, inc);
  }
}

// per-device side stream and events of the copy-engine all-gather
struct CeState { cudaStream_t stream; cudaEvent_t ready, done; };
CeState* ce_state() {
  static CeState st[64];
  static bool made[64] = {false};
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return nullptr;
  if (!made[dev]) {
    if (cudaStreamCreateWithFlags(&st[dev].stream, cudaStreamNonBlocking) != cudaSuccess) return nullptr;
    if (cudaEventCreateWithFlags(&st[dev].ready, cudaEventDisableTiming) != cudaSuccess) return nullptr;
    if (cudaEventCreateWithFlags(&st[dev].done, cudaEventDisableTiming) != cudaSuccess) return nullptr;
    made[dev] = true;
  }
  return &st[dev];
}

void bind_ctx() {
  static thread_local bool ctx_bound = false;
  if (!ctx_bound) {
    cudaFree(0);
    ctx_bound = true;
  }
}
}  // namespace

// All-gather -> GEMM in one kernel.  C[M,N] = gather(x)[M,K] . op(B)^T; this rank contributes
// x_local [M/n, K] (row stride ld_x), rows [rank*M/n, ...).  gather_ptrs[r] = rank r's gather buffer
// [M,K] contiguous (peer pointers for r != rank); after the kernel gather_ptrs[rank] holds the whole
// gathered operand.  flag_ptrs[r] = rank r's block counters [M/128] (zeroed once); ag_target =
// (number of calls that used these counters, this one included) * 6.  n_comm > 0: that many mover
// CTAs inside the kernel push the rows; n_comm < 0: copy-engine transfers on a side stream bring
// them instead and every SM runs GEMM tiles.
// M must be a multiple of 128 * n_ranks.  gather_ptrs / flag_ptrs are host arrays of n_ranks pointers.
extern "C" int lb_gemm_ag(const void* B, void* C, int M, int N, int K, long long ldb, long long ldc, int b_mn,
                          int n_ranks, int rank, const void* x_local, long long ld_x, void* const* gather_ptrs,
                          void* const* flag_ptrs, unsigned int ag_target, int n_comm, void* stream) {
  if (M <= 0 || N <= 0 || K <= 0 || n_ranks < 2 || n_ranks > MAX_RANKS) return LB_ERR_SHAPE;
  if ((ldb % 8) || (ldc % 8) || (N % 8) || (K % 8) || (ld_x % 8) || (M % (BM * n_ranks))) return LB_ERR_SHAPE;
  bind_ctx();
  CUtensorMap ta, tb, town;
  int rc = make_map(&ta, gather_ptrs[rank], (uint64_t)K, (uint64_t)M, (uint64_t)K, BK, BM);
  if (rc) return rc;
  if (!b_mn) rc = make_map(&tb, B, (uint64_t)K, (uint64_t)N, (uint64_t)ldb, BK, BN);
  else       rc = make_map(&tb, B, (uint64_t)N, (uint64_t)K, (uint64_t)ldb, 64, BK);
  if (rc) return rc;
  rc = make_map(&town, x_local, (uint64_t)K, (uint64_t)(M / n_ranks), (uint64_t)ld_x, BK, BM);
  if (rc) return rc;
  const int sms = init_sms();
  GemmParams p;
  p.M = M; p.N = N; p.K = K; p.ldc = ldc; p.a_mn = 0; p.b_mn = b_mn;
  p.tiles_m = M / BM;
  p.tiles_n = (N + BN - 1) / BN;
  p.num_tiles = p.tiles_m * p.tiles_n;
  p.num_kb = (K + BK - 1) / BK;
  CommParams cp;
  memset(&cp, 0, sizeof(cp));
  cp.n_ranks = n_ranks; cp.rank = rank; cp.rows_per_rank = M / n_ranks; cp.blocks_per_rank = cp.rows_per_rank / BM;
  const bool copy_engine = n_comm < 0;          // rows travel by copy-engine transfers issued here, not by mover CTAs
  if (copy_engine) n_comm = 0;
  else if (n_comm < 1) n_comm = 1;
  if (n_comm > sms / 2) n_comm = sms / 2;
  cp.n_comm = n_comm; cp.ag_target = ag_target; cp.wait_ns = g_lb_flag_wait_ns;
  cp.x_local = (const bf16*)x_local; cp.ld_x = ld_x;
  for (int r = 0; r < n_ranks; r++) { cp.gather[r] = (bf16*)gather_ptrs[r]; cp.ag_flags[r] = (unsigned int*)flag_ptrs[r]; }
  CeState* ce = nullptr;
  if (copy_engine) {
    // Side stream: one peer copy per destination and quarter of this rank's rows (the copy engines
    // reach about twice the NVLink rate that SM-issued stores were measured at here), each followed by
    // a few-thread kernel that raises the arrival counters of the copied 128-row blocks by the same
    // amount the mover warps would.  The GEMM kernel below starts at once on all SMs and consumes the
    // blocks as their counters arrive; the calling stream is made to wait for the copies afterwards,
    // so x_local may be reused by whatever is enqueued next.
    ce = ce_state();
    if (ce == nullptr) return LB_ERR_LAUNCH;
    cudaStream_t main = (cudaStream_t)stream;
    cudaEventRecord(ce->ready, main);
    cudaStreamWaitEvent(ce->stream, ce->ready, 0);
    const int bpr = cp.blocks_per_rank;
    const int parts = bpr >= 4 ? 4 : 1;
    const bf16* xl = (const bf16*)x_local;
    for (int pt = 0; pt < parts; pt++) {
      const int b0 = (int)((long long)bpr * pt / parts), b1 = (int)((long long)bpr * (pt + 1) / parts);
      const size_t r0 = (size_t)b0 * BM, nrows = (size_t)(b1 - b0) * BM;
      for (int j = 1; j <= n_ranks; j++) {                      // peers first, the local copy last
        const int dst = (rank + j) % n_ranks;
        bf16* d = cp.gather[dst] + ((size_t)rank * cp.rows_per_rank + r0) * K;
        cudaMemcpy2DAsync(d, (size_t)K * 2, xl + r0 * ld_x, (size_t)ld_x * 2, (size_t)K * 2, nrows, cudaMemcpyDeviceToDevice,
                          ce->stream);
        if (dst != rank)
          ag_flag_bump_kernel<<<1, 128, 0, ce->stream>>>(cp.ag_flags[dst] + rank * bpr + b0, b1 - b0, (unsigned)MOVER_WARPS);
      }
    }
    cudaEventRecord(ce->done, ce->stream);
  }
  int n_gemm = sms - n_comm;
  if (n_gemm > p.num_tiles) n_gemm = p.num_tiles;
  gemm_bf16_kernel<1><<<n_comm + n_gemm, NUM_THREADS, SMEM_BYTES, (cudaStream_t)stream>>>(ta, tb, town, (bf16*)C, p, cp);
  LB_CHECK_LAUNCH();
  if (ce) cudaStreamWaitEvent((cudaStream_t)stream, ce->done, 0);
  return LB_OK;
}

// GEMM -> reduce-scatter in one kernel.  Every rank computes A[M,K_local] . op(B)^T; rank r ends
// with out[M/n, N] = sum over ranks of rows [r*M/n, ...).  recv_ptrs[r] = rank r's receive area
// [n_ranks][M/n][N] bf16, flag_ptrs[r] = rank r's counters [n_ranks][M/n/128] (zeroed once);
// rs_target = previous target of these counters + 4 * ceil(N/256).
extern "C" int lb_gemm_rs(const void* A, const void* B, int M, int N, int K, long long lda, long long ldb, int b_mn,
                          int n_ranks, int rank, void* const* recv_ptrs, void* const* flag_ptrs, unsigned int rs_target,
                          void* out, long long ld_out, void* stream) {
  if (M <= 0 || N <= 0 || K <= 0 || n_ranks < 2 || n_ranks > MAX_RANKS) return LB_ERR_SHAPE;
  if ((lda % 8) || (ldb % 8) || (ld_out % 8) || (N % 8) || (M % (BM * n_ranks))) return LB_ERR_SHAPE;
  bind_ctx();
  CUtensorMap ta, tb;
  int rc = make_map(&ta, A, (uint64_t)K, (uint64_t)M, (uint64_t)lda, BK, BM);
  if (rc) return rc;
  if (!b_mn) rc = make_map(&tb, B, (uint64_t)K, (uint64_t)N, (uint64_t)ldb, BK, BN);
  else       rc = make_map(&tb, B, (uint64_t)N, (uint64_t)K, (uint64_t)ldb, 64, BK);
  if (rc) return rc;
  const int sms = init_sms();
  GemmParams p;
  p.M = M; p.N = N; p.K = K; p.ldc = N; p.a_mn = 0; p.b_mn = b_mn;
  p.tiles_m = M / BM;
  p.tiles_n = (N + BN - 1) / BN;
  p.num_tiles = p.tiles_m * p.tiles_n;
  p.num_kb = (K + BK - 1) / BK;
  CommParams cp;
  memset(&cp, 0, sizeof(cp));
  cp.n_ranks = n_ranks; cp.rank = rank; cp.rows_per_rank = M / n_ranks; cp.blocks_per_rank = cp.rows_per_rank / BM;
  cp.rs_target = rs_target; cp.wait_ns = g_lb_flag_wait_ns;
  for (int r = 0; r < n_ranks; r++) { cp.recv[r] = (bf16*)recv_ptrs[r]; cp.rs_flags[r] = (unsigned int*)flag_ptrs[r]; }
  cp.out = (bf16*)out; cp.ld_out = ld_out;
  int grid = p.num_tiles < sms ? p.num_tiles : sms;
  gemm_bf16_kernel<2><<<grid, NUM_THREADS, SMEM_BYTES_RS, (cudaStream_t)stream>>>(ta, tb, ta, nullptr, p, cp);
  LB_CHECK_LAUNCH();
  return LB_OK;
}
