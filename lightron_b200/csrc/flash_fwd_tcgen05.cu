// FlashAttention forward on the 5th-generation tensor cores (sm_100a), head_dim 64 or 128.
//
// One CTA owns 256 consecutive queries of one (batch, head): two 128-row tiles that ping-pong on
// the tensor pipe.  Per 128-key block:
//     S_t = Q_t K^T          tcgen05.mma, 128x128xd, operands in 128B-swizzled smem (TMA), D in TMEM
//     softmax(S_t)           one thread per query row reads its row straight from TMEM
//                            (tcgen05.ld), so max / sum need no shuffles; P_t goes back to TMEM as
//                            packed bf16 pairs (tcgen05.st)
//     O_t (+)= P_t V         tcgen05.mma with the A operand in TMEM, 128 x d x 128, V is the MN-major
//                            B operand as it sits in memory
// P never touches shared memory: with P staged there the kernel was bound by shared-memory
// bandwidth (128 B/clk: the P stores, the A-operand reads of P V and of Q K^T, the TMA writes),
// measured as tcgen05.mma issue blocking for 400 / 620 cycles per S / P V group at head_dim 64.
// O_t stays in TMEM for the whole key loop; when a row maximum grows the softmax threads rescale
// it in place (tcgen05.ld / st) before the next P V is issued.
// Warp roles (384 threads): warp 0 TMA producer, warps 1 / 2 MMA issuers of tile 0 / 1 (warp 1
// owns the TMEM allocation), warp 3 idle, warps 4-7 softmax of tile 0, warps 8-11 softmax of tile 1.
// The two tiles run half a period apart (tile 1 starts late on purpose): the exponentials of one
// then overlap the loads, maxima and waits of the other instead of queueing on the same MUFU unit.  While one tile is in softmax the tensor pipe
// works on the other.  Layout / masking conventions are those of flash_attn.cu.
// All waits are bounded; on expiry a status word is set and the CTA drains and frees its TMEM.
#include <string.h>
#include "tcgen05.cuh"
#include "comm.cuh"

static __device__ unsigned int g_fa_status[4] = {0, 0, 0, 0};

// Developer instrumentation (build with -DLB_FA_PROFILE): cycles that lane 0 of every softmax warp
// spends in each phase of the key-block loop, summed over the grid.  lb_flash_prof() reads and clears.
#ifdef LB_FA_PROFILE
static __device__ unsigned long long g_fa_prof[16];
#define FA_T(i) const long long tp##i = clock64()
#define FA_ACC(slot, a, b) prof[slot] += (unsigned long long)(tp##b - tp##a)
#else
#define FA_T(i)
#define FA_ACC(slot, a, b)
#endif

namespace {
using namespace bw;

// Context-parallel extension ("all-gather KV inside the attention kernel"): the K/V operand is a
// gather buffer [B, S_full, hkv*d] in peer-visible memory that every rank of the CP group fills
// by PUSHING its own zig-zag chunks (rank r owns sequence chunks r and 2c-1-r) with coalesced
// peer stores from `n_mov` mover CTAs of this same kernel, counting each 128-key block in the
// destination's flag word.  The attention CTAs gate every 128-key block on its flag, so the
// exchange overlaps the softmax / MMA work on blocks that have already arrived.
constexpr int FA_MAX_RANKS = 8;
constexpr int FA_FWD_THREADS = 384;
struct FaPush {
  int n_mov, n_ranks, rank, chunk_rows, row_elems;   // row_elems = hkv * d
  const bf16 *k_src, *v_src;                         // this rank's [B, 2*chunk_rows, hkv, d], token strides below
  long long k_ts, v_ts;
  bf16* k_dst[FA_MAX_RANKS];                         // rank r's gather buffers [B, S_full, hkv*d]
  bf16* v_dst[FA_MAX_RANKS];
  unsigned int* flags[FA_MAX_RANKS];                 // rank r's block counters [B][S_full / 128]
};
struct FaFwdParams {
  bf16* o;
  float* lse;
  int B, Sq, Sk, hq, hkv;
  long long o_ts;
  float scale;
  int causal;
  int kv_brows;                  // rows between consecutive batches in the K/V tensor maps (>= Sk)
  const unsigned int* kv_flags;  // null, or this rank's block counters [B][kv_brows / 128]
  unsigned int flag_target;
  int tiles_x;                   // query tiles (256 rows) per (batch, head)
  unsigned long long wait_ns;    // limit of a wait on a key block's arrival flag
};

// 2^x on the FMA pipe: round to the nearest integer with the 1.5 * 2^23 trick, a degree-4 polynomial
// for the fraction in [-0.5, 0.5] (relative error 6e-5, far below the bf16 rounding of P), and
// the integer part added to the exponent field.  Inputs below -126 (masked scores are -inf) give ~0.
__device__ __forceinline__ float exp2_poly(float x) {
  x = fmaxf(x, -126.f);
  const float t = x + 12582912.f;
  const float f = x - (t - 12582912.f);
  float p = fmaf(f, 9.6181291e-3f, 5.5504109e-2f);
  p = fmaf(p, f, 2.4022651e-1f);
  p = fmaf(p, f, 6.9314718e-1f);
  p = fmaf(p, f, 1.0f);
  return __int_as_float(__float_as_int(p) + (__float_as_int(t) << 23));
}
// Off by default: measured at B8 S2048 32q/4kv d64, every 2nd / 4th / 8th pair on the polynomial gave
// 0.394 / 0.333 / 0.335 ms against 0.316 ms with the MUFU alone (the extra FMA-pipe instructions cost
// more issue slots than the MUFU cycles they free).
#ifndef LB_FA_POLY_EVERY
#define LB_FA_POLY_EVERY 0
#endif

template <int D>
struct FaCfg {
  static constexpr int BM = 128, BN = 128;
  static constexpr int KS = (D == 64) ? 3 : 2;
  static constexpr int VS = (D == 64) ? 3 : 1;
  static constexpr int ATOMS = D / 64;
  static constexpr int ATOM_BYTES = 128 * 128;          // 128 rows x 128 B
  static constexpr int TILE_BYTES = ATOMS * ATOM_BYTES; // one Q / K / V tile
  // TMEM columns: S_t fp32 [128], O_t fp32 [D], P_t packed bf16 [64].  With head_dim 64 all six
  // regions fit in the 512 columns and P never touches shared memory.  With head_dim 128 S and O
  // fill the 512 columns: P_t is staged in shared memory instead (letting P_t take columns of S_t
  // was measured slower: S_t of the next key block then has to queue behind P_t V).
  static constexpr bool P_TMEM = (D == 64);
  static constexpr int COL_S = 0, COL_O = 256, COL_P = 384;
  static constexpr int P_STRIDE = 64;
  static constexpr int P_BYTES = 2 * ATOM_BYTES;        // 128 x 128 bf16 (shared-memory variant)
  static constexpr int OFF_Q = 0;
  static constexpr int OFF_K = OFF_Q + 2 * TILE_BYTES;
  static constexpr int OFF_V = OFF_K + KS * TILE_BYTES;
  static constexpr int OFF_P = OFF_V + VS * TILE_BYTES;
  static constexpr int OFF_BAR = OFF_P + (P_TMEM ? 0 : 2 * P_BYTES);
  static constexpr int SMEM = OFF_BAR + 256 + 1024;
  static constexpr int NBAR = 1 + 2 * KS + 2 * VS + 8;
};

template <int D>
__global__ void __launch_bounds__(FA_FWD_THREADS, 1)
fa_fwd_tc_kernel(const __grid_constant__ CUtensorMap tq, const __grid_constant__ CUtensorMap tk,
                 const __grid_constant__ CUtensorMap tv, const FaFwdParams p, const FaPush push) {
  using C = FaCfg<D>;
  if ((int)blockIdx.x < push.n_mov) {
    // ------------------------------- K/V mover CTAs -------------------------------
    // unit = (destination rank, batch, which of this rank's two chunks, 128-row block, K or V)
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, nwarps = blockDim.x >> 5;
    const int bpc = push.chunk_rows / 128;
    const int fpb = (2 * push.n_ranks * push.chunk_rows) / 128;       // flag words per batch
    const int units = push.n_ranks * p.B * 2 * bpc * 2;
    const int vec_per_row = push.row_elems / 8;
    for (int u = blockIdx.x; u < units; u += push.n_mov) {
      int t = u;
      const int kv = t & 1; t >>= 1;
      const int blk = t % bpc; t /= bpc;
      const int half = t & 1; t >>= 1;
      const int b = t % p.B; t /= p.B;
      const int dst = (push.rank + 1 + t) % push.n_ranks;
      const int chunk = half ? 2 * push.n_ranks - 1 - push.rank : push.rank;
      const long long lrow0 = (long long)b * 2 * push.chunk_rows + half * push.chunk_rows + blk * 128;
      const long long grow0 = (long long)b * fpb * 128 + (long long)chunk * push.chunk_rows + blk * 128;
      const bf16* src = kv ? push.v_src : push.k_src;
      const long long ts = kv ? push.v_ts : push.k_ts;
      bf16* dstp = (kv ? push.v_dst[dst] : push.k_dst[dst]) + grow0 * push.row_elems;
      // every warp copies its share of the block's rows, fences and counts by itself: while one warp
      // sits in its fence the others keep streaming
      for (int r = warp; r < 128; r += nwarps) {
        const uint4* sp = reinterpret_cast<const uint4*>(src + (lrow0 + r) * ts);
        uint4* dp = reinterpret_cast<uint4*>(dstp + (long long)r * push.row_elems);
        for (int v0 = 0; v0 < vec_per_row; v0 += 128) {
          uint4 a[4];
#pragma unroll
          for (int j = 0; j < 4; j++) if (v0 + j * 32 + lane < vec_per_row) a[j] = sp[v0 + j * 32 + lane];
#pragma unroll
          for (int j = 0; j < 4; j++) if (v0 + j * 32 + lane < vec_per_row) dp[v0 + j * 32 + lane] = a[j];
        }
      }
      __threadfence_system();
      __syncwarp();
      if (lane == 0)
        lbcomm::red_release_sys_add(push.flags[dst] + (grow0 >> 7), 1u);
    }
    return;
  }
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~(uintptr_t)1023);
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + C::OFF_BAR);
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + C::NBAR);
  __shared__ int s_abort[2];     // {abort, extra wait in ms}: see bw::mbar_wait

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const uint32_t sbase = smem_u32(smem);
  const uint32_t bar0 = smem_u32(bars);
  // barrier map
  const uint32_t q_full = bar0;
  auto k_full = [&](int s) { return bar0 + 8u * (1 + s); };
  auto k_empty = [&](int s) { return bar0 + 8u * (1 + C::KS + s); };
  auto v_full = [&](int s) { return bar0 + 8u * (1 + 2 * C::KS + s); };
  auto v_empty = [&](int s) { return bar0 + 8u * (1 + 2 * C::KS + C::VS + s); };
  const uint32_t bar1 = bar0 + 8u * (1 + 2 * C::KS + 2 * C::VS);
  auto s_full = [&](int t) { return bar1 + 8u * t; };
  auto p_full = [&](int t) { return bar1 + 8u * (2 + t); };
  auto pv_done = [&](int t) { return bar1 + 8u * (4 + t); };
  auto s_free = [&](int t) { return bar1 + 8u * (6 + t); };

  // 1-D grid: movers first (they must be resident before anything waits for data), then the
  // (query tile, head, batch) CTAs with the tile index fastest
  const int cid = (int)blockIdx.x - push.n_mov;
  const int mblk = p.tiles_x - 1 - cid % p.tiles_x;   // late (long) causal rows first
  const int h = (cid / p.tiles_x) % p.hq, b = cid / (p.tiles_x * p.hq);
  const int hk = h / (p.hq / p.hkv);
  const int m0 = mblk * 2 * C::BM;
  const int off = p.Sk - p.Sq;
  const int kv_blocks = (p.Sk + C::BN - 1) / C::BN;
  int nb[2];
#pragma unroll
  for (int t = 0; t < 2; t++) {
    const int r0 = m0 + t * C::BM;
    int n = kv_blocks;
    if (p.causal) n = min(n, (r0 + C::BM - 1 + off) / C::BN + 1);
    nb[t] = (r0 < p.Sq) ? n : 0;
  }
  const int nb_max = max(nb[0], nb[1]);

  if (threadIdx.x == 0) {
    s_abort[0] = 0;
    s_abort[1] = p.kv_flags ? wait_extra_ms(p.wait_ns) : 0;
    mbar_init(q_full, 1);
    for (int s = 0; s < C::KS; s++) { mbar_init(k_full(s), 1); mbar_init(k_empty(s), 2); }
    for (int s = 0; s < C::VS; s++) { mbar_init(v_full(s), 1); mbar_init(v_empty(s), 2); }
    for (int t = 0; t < 2; t++) { mbar_init(s_full(t), 1); mbar_init(p_full(t), 128); mbar_init(pv_done(t), 1); mbar_init(s_free(t), 128); }
    mbar_init_fence();
    prefetch_tmap(&tq); prefetch_tmap(&tk); prefetch_tmap(&tv);
  }
  if (warp == 1) tmem_alloc(smem_u32(tmem_slot), 512);
  fence_before();
  __syncthreads();
  fence_after();
  const uint32_t tmem_base = *tmem_slot;
  volatile int* abort_flag = s_abort;

  // (with LB_FA_SETMAXNREG) warps 0-3 (loads, MMA issue) hand registers to the eight softmax warps,
  // which hold a 128-column row of scores each
#ifdef LB_FA_SETMAXNREG
#define FA_REG_DEC() asm volatile("setmaxnreg.dec.sync.aligned.u32 96;")
#define FA_REG_INC() asm volatile("setmaxnreg.inc.sync.aligned.u32 200;")
#else
#define FA_REG_DEC()
#define FA_REG_INC()
#endif
  if (warp == 0) {
    FA_REG_DEC();
    // ------------------------------- TMA producer -------------------------------
    if (lane == 0 && nb_max > 0) {
      mbar_expect_tx(q_full, 2 * C::TILE_BYTES);
#pragma unroll
      for (int t = 0; t < 2; t++)
#pragma unroll
        for (int a = 0; a < C::ATOMS; a++)
          tma_load_2d(sbase + C::OFF_Q + t * C::TILE_BYTES + a * C::ATOM_BYTES, &tq, h * D + a * 64,
                      b * p.Sq + m0 + t * C::BM, q_full);
      bool ok = true;
      for (int j = 0; j < nb_max && ok; j++) {
        const int ks = j % C::KS, vs = j % C::VS;
        if (!mbar_wait(k_empty(ks), (((uint32_t)(j / C::KS)) & 1u) ^ 1u, abort_flag)) { ok = false; break; }
        if (p.kv_flags) {
          // this 128-key block is pushed by its owner: wait for its counter, then order the
          // peer's generic-proxy writes before the TMA (async proxy) reads
          if (!lbcomm::flag_wait_ge(p.kv_flags + (long long)b * (p.kv_brows >> 7) + j, p.flag_target, p.wait_ns)) { *abort_flag = 1; ok = false; break; }
          asm volatile("fence.proxy.async;" ::: "memory");
        }
        mbar_expect_tx(k_full(ks), C::TILE_BYTES);
#pragma unroll
        for (int a = 0; a < C::ATOMS; a++)
          tma_load_2d(sbase + C::OFF_K + ks * C::TILE_BYTES + a * C::ATOM_BYTES, &tk, hk * D + a * 64,
                      b * p.kv_brows + j * C::BN, k_full(ks));
        if (!mbar_wait(v_empty(vs), (((uint32_t)(j / C::VS)) & 1u) ^ 1u, abort_flag)) { ok = false; break; }
        mbar_expect_tx(v_full(vs), C::TILE_BYTES);
#pragma unroll
        for (int a = 0; a < C::ATOMS; a++)
          tma_load_2d(sbase + C::OFF_V + vs * C::TILE_BYTES + a * C::ATOM_BYTES, &tv, hk * D + a * 64,
                      b * p.kv_brows + j * C::BN, v_full(vs));
      }
      if (!ok) atomicExch(&g_fa_status[0], 1u);
    }
  } else if (warp == 1 || warp == 2) {
    FA_REG_DEC();
    // ------------------------------- MMA issuers -------------------------------
    // One issuing thread per query tile.  A tcgen05.mma costs its issuer 60-90 cycles whatever its
    // size (measured: 370 cycles for the four 128x128x16 of one S, 500 for the eight 128x64x16 of
    // one P V), so a single thread feeding both tiles was the bottleneck of the whole kernel; two
    // threads issue side by side and each follows the fixed order of its own tile with blocking
    // waits: S(0); then per key block S(j+1) as soon as the softmax threads hold S(j) in registers,
    // and P(j) V as soon as P(j) is in TMEM (or, head_dim 128, in shared memory).
    // A K / V stage is free once BOTH tiles have used it, so each thread arrives on the stage's
    // empty barrier for every block, also for blocks its own tile does not need.
    const int t = warp - 1;
    if (lane == 0 && nb_max > 0) {
      const uint32_t idesc_s = make_idesc(C::BM, C::BN, 0, 0);
      const uint32_t idesc_o = make_idesc(C::BM, D, 0, 1);
      // descriptor bases; a stage / k-step only changes the 16-byte-granular start address
      const uint64_t qa = make_desc(sbase + C::OFF_Q + t * C::TILE_BYTES, 16, 1024);
      const uint64_t dk0 = make_desc(sbase + C::OFF_K, 16, 1024);
      const uint64_t dv0 = make_desc(sbase + C::OFF_V, C::ATOM_BYTES, 1024);
      const uint32_t s_dst = tmem_base + C::COL_S + t * C::BN;
      const uint32_t o_dst = tmem_base + C::COL_O + t * D;
      const uint32_t pa = tmem_base + C::COL_P + t * C::P_STRIDE;          // 8 columns per K = 16 slice
      const uint64_t dp0 = make_desc(sbase + C::OFF_P + t * C::P_BYTES, 16, 1024);
      const int n_my = nb[t];
      bool ok = mbar_wait(q_full, 0, abort_flag);
      auto issue_s = [&](int j) -> bool {             // S(j) = Q K(j)^T, then release K(j)'s stage
        const int ks = j % C::KS;
        if (!mbar_wait(k_full(ks), ((uint32_t)(j / C::KS)) & 1u, abort_flag)) return false;
        fence_after();
        const uint64_t ka = dk0 + (uint64_t)((ks * C::TILE_BYTES) >> 4);
#pragma unroll
        for (int s = 0; s < D / 16; s++) {
          const uint64_t o = (uint64_t)(((s >> 2) * C::ATOM_BYTES + (s & 3) * 32) >> 4);
          umma_bf16(s_dst, qa + o, ka + o, idesc_s, s ? 1u : 0u);
        }
        umma_commit(s_full(t));
        umma_commit(k_empty(ks));
        return true;
      };
      auto issue_pv = [&](int j) -> bool {            // O += P(j) V(j), then release V(j)'s stage
        const int vs = j % C::VS;
        if (!mbar_wait(p_full(t), (uint32_t)j & 1u, abort_flag)) return false;
        if (!mbar_wait(v_full(vs), ((uint32_t)(j / C::VS)) & 1u, abort_flag)) return false;
        fence_after();
        const uint64_t va = dv0 + (uint64_t)((vs * C::TILE_BYTES) >> 4);
        if (C::P_TMEM) {
          umma_bf16_ta(o_dst, pa, va, idesc_o, j ? 1u : 0u);
#pragma unroll
          for (int s = 1; s < C::BN / 16; s++)
            umma_bf16_ta(o_dst, pa + 8u * s, va + (uint64_t)((s * 2048) >> 4), idesc_o, 1u);
        } else {
          umma_bf16(o_dst, dp0, va, idesc_o, j ? 1u : 0u);
#pragma unroll
          for (int s = 1; s < C::BN / 16; s++)
            umma_bf16(o_dst, dp0 + (uint64_t)(((s >> 2) * C::ATOM_BYTES + (s & 3) * 32) >> 4), va + (uint64_t)((s * 2048) >> 4),
                      idesc_o, 1u);
        }
        umma_commit(pv_done(t));
        umma_commit(v_empty(vs));
        return true;
      };
      // stagger: tile 1 starts once tile 0 holds its first S in registers (two tiles marching in
      // step were measured to spend 2300 cycles per block together in the exponentials and then
      // idle together; half a period apart each has the MUFU unit to itself)
      if (ok && t == 1 && nb[0] > 0 && n_my > 0) ok = mbar_wait(s_free(0), 0u, abort_flag);
      if (ok && n_my > 0) ok = issue_s(0);
      for (int j = 0; j < n_my && ok; j++) {
        if (j + 1 < n_my) {
          ok = mbar_wait(s_free(t), (uint32_t)j & 1u, abort_flag);
          if (ok) ok = issue_s(j + 1);
        }
        if (ok) ok = issue_pv(j);
      }
      // blocks that only the other tile needs: keep the stage rings in step
      for (int j = n_my; j < nb_max && ok; j++) {
        ok = mbar_wait(k_full(j % C::KS), ((uint32_t)(j / C::KS)) & 1u, abort_flag);
        if (ok) mbar_arrive(k_empty(j % C::KS));
        if (ok) ok = mbar_wait(v_full(j % C::VS), ((uint32_t)(j / C::VS)) & 1u, abort_flag);
        if (ok) mbar_arrive(v_empty(j % C::VS));
      }
      if (!ok) atomicExch(&g_fa_status[0], 2u);
    }
  } else if (warp == 3) {
    FA_REG_DEC();
  } else {
    // ------------------------------- softmax warps -------------------------------
    FA_REG_INC();
    const int t = (warp - 4) >> 2;
    const int quad = warp & 3;
    const int rit = quad * 32 + lane;              // row inside the tile
    const int row = m0 + t * C::BM + rit;          // query index inside the sequence
    const uint32_t lane_addr = tmem_base + ((uint32_t)(quad * 32) << 16);
    const uint32_t ts_addr = lane_addr + C::COL_S + t * C::BN;
    const uint32_t to_addr = lane_addr + C::COL_O + t * D;
    const uint32_t tp_addr = lane_addr + C::COL_P + t * C::P_STRIDE;
    uint8_t* sP = smem + C::OFF_P + t * C::P_BYTES;
    const float sl2 = p.scale * 1.4426950408889634f;
    constexpr int POLY_EVERY = (D == 64) ? LB_FA_POLY_EVERY : 0;   // head_dim 128 has twice the MMA work per exponential
    float m_i = -INFINITY, l_i = 0.f;
    bool ok = true;
    const int n_my = nb[t];
#ifdef LB_FA_PROFILE
    unsigned long long prof[8] = {0, 0, 0, 0, 0, 0, 0, 0};
#endif
    for (int j = 0; j < n_my; j++) {
      FA_T(0);
      if (!mbar_wait(s_full(t), (uint32_t)j & 1u, abort_flag)) { ok = false; break; }
      fence_after();
      FA_T(1);
      uint32_t r[128];
      const int c0 = j * C::BN;
      const int warp_row0 = m0 + t * C::BM + quad * 32;
      const bool need_mask = (c0 + C::BN > p.Sk) || (p.causal && (c0 + C::BN - 1 > warp_row0 + off));
      const int lim = (p.causal ? min(p.Sk - 1, row + off) : p.Sk - 1) - c0;   // last visible column of this block
      // the row arrives in two halves so that the maximum of the first overlaps the second load;
      // four independent chains keep the 128 comparisons from serialising on their latency
      float mx4[4] = {-INFINITY, -INFINITY, -INFINITY, -INFINITY};
      tmem_ld32(ts_addr, r);
      tmem_ld32(ts_addr + 32, r + 32);
      tmem_ld_wait();
      tmem_ld32(ts_addr + 64, r + 64);
      tmem_ld32(ts_addr + 96, r + 96);
#pragma unroll
      for (int half = 0; half < 2; half++) {
        if (half == 1) {
          tmem_ld_wait();
          fence_before();
          mbar_arrive(s_free(t));                     // S_t may be overwritten by the next key block
        }
        if (need_mask) {
#pragma unroll
          for (int i = half * 64; i < half * 64 + 64; i++) {
            if (i > lim) r[i] = 0xff800000u;           // -inf
            mx4[i & 3] = fmaxf(mx4[i & 3], __uint_as_float(r[i]));
          }
        } else {
#pragma unroll
          for (int i = half * 64; i < half * 64 + 64; i++) mx4[i & 3] = fmaxf(mx4[i & 3], __uint_as_float(r[i]));
        }
      }
      const float mx = fmaxf(fmaxf(mx4[0], mx4[1]), fmaxf(mx4[2], mx4[3]));
      FA_T(2);
      // Lazy reference maximum: keep the old one unless the new maximum is more than 2^8 above
      // it, so that O and l rarely need rescaling (values stay below 2^8 relative to it).
      float m_new = fmaxf(m_i, mx);
      if (m_i != -INFINITY && (m_new - m_i) * sl2 <= 8.f) m_new = m_i;
      const float m_s = (m_new == -INFINITY) ? 0.f : m_new * sl2;
      const float corr = (m_i == -INFINITY) ? 0.f : exp2f(m_i * sl2 - m_s);
      FA_T(3);
      // exponentials; P goes back to TMEM as packed bf16 pairs (column c holds keys 2c, 2c+1), 32
      // columns per store so that the first store is in flight while the second half is computed.
      // The first half is computed BEFORE waiting for the previous P V (which still reads the P
      // columns and owns O): its 64 exponentials overlap the tail of that MMA.
      float rs2[2] = {0.f, 0.f};
#pragma unroll
      for (int hh = 0; hh < 2; hh++) {
        uint32_t pr[32];
#pragma unroll
        for (int c = 0; c < 32; c++) {
          const int i = hh * 64 + c * 2;
          // the MUFU unit (16 exponentials per clock per SM) is this kernel's ceiling at small head
          // dimensions: every POLY_EVERY-th pair is evaluated on the FMA pipe instead
          float e0, e1;
          if (POLY_EVERY > 0 && (c % (POLY_EVERY > 0 ? POLY_EVERY : 1)) == 0) {
            e0 = exp2_poly(fmaf(__uint_as_float(r[i]), sl2, -m_s));
            e1 = exp2_poly(fmaf(__uint_as_float(r[i + 1]), sl2, -m_s));
          } else {
            e0 = exp2f(fmaf(__uint_as_float(r[i]), sl2, -m_s));
            e1 = exp2f(fmaf(__uint_as_float(r[i + 1]), sl2, -m_s));
          }
          rs2[c & 1] += e0 + e1;
          bf162 pk = __floats2bfloat162_rn(e0, e1);
          pr[c] = *reinterpret_cast<uint32_t*>(&pk);
        }
        if (hh == 0 && j > 0) {
          // previous P V finished: O is stable and the P columns may be overwritten
          if (!mbar_wait(pv_done(t), (uint32_t)(j - 1) & 1u, abort_flag)) { ok = false; }
          fence_after();
          if (ok && __any_sync(0xffffffffu, m_new != m_i)) {
#pragma unroll 1
            for (int c = 0; c < D / 32; c++) {
              uint32_t o[32];
              tmem_ld32(to_addr + c * 32, o);
              tmem_ld_wait();
#pragma unroll
              for (int i = 0; i < 32; i++) o[i] = __float_as_uint(__uint_as_float(o[i]) * corr);
              tmem_st32(to_addr + c * 32, o);
            }
            tmem_st_wait();
          }
        }
        if (C::P_TMEM) {
          tmem_st32(tp_addr + hh * 32, pr);
        } else {
          // keys hh*64 .. +63 of this row are 128 bytes: one row of swizzle atom hh
#pragma unroll
          for (int c16 = 0; c16 < 8; c16++)
            *reinterpret_cast<uint4*>(sP + hh * C::ATOM_BYTES + sw128_off(rit, c16)) =
                make_uint4(pr[c16 * 4], pr[c16 * 4 + 1], pr[c16 * 4 + 2], pr[c16 * 4 + 3]);
        }
      }
      if (!ok) break;
      if (C::P_TMEM) tmem_st_wait(); else fence_proxy_async_smem();
      l_i = l_i * corr + (rs2[0] + rs2[1]);
      m_i = m_new;
      FA_T(4);
      fence_before();
      mbar_arrive(p_full(t));
      FA_T(5);
      FA_ACC(0, 0, 1); FA_ACC(1, 1, 2); FA_ACC(2, 2, 3); FA_ACC(3, 3, 4); FA_ACC(4, 4, 5);
#ifdef LB_FA_PROFILE
      prof[5] += 1;
#endif
    }
#ifdef LB_FA_PROFILE
    if (lane == 0)
      for (int i = 0; i < 8; i++) atomicAdd(&g_fa_prof[i], prof[i]);
#endif
    if (ok && n_my > 0) {
      if (!mbar_wait(pv_done(t), (uint32_t)(n_my - 1) & 1u, abort_flag)) ok = false;
    }
    if (ok && n_my > 0) {
      fence_after();
      const float inv = l_i > 0.f ? 1.f / l_i : 0.f;
      bf16* orow = p.o + ((long long)b * p.Sq + row) * p.o_ts + (long long)h * D;
#pragma unroll 1
      for (int c = 0; c < D / 32; c++) {
        uint32_t r[32];
        tmem_ld32(to_addr + c * 32, r);
        tmem_ld_wait();
        if (row < p.Sq) {
          float f[32];
#pragma unroll
          for (int i = 0; i < 32; i++) f[i] = __uint_as_float(r[i]) * inv;
#pragma unroll
          for (int g = 0; g < 4; g++) *reinterpret_cast<uint4*>(orow + c * 32 + g * 8) = pack8(f + g * 8);
        }
      }
      if (row < p.Sq)
        p.lse[((long long)b * p.hq + h) * p.Sq + row] = (l_i > 0.f) ? m_i * p.scale + logf(l_i) : -INFINITY;
    }
    if (!ok && lane == 0) atomicExch(&g_fa_status[0], 3u);
  }

  fence_before();
  __syncthreads();
  if (warp == 1) {
    fence_after();
    tmem_dealloc(tmem_base, 512);
  }
}

template <int D>
int launch_fa_fwd(const void* q, const void* k, const void* v, FaFwdParams p, const FaPush& push, long long q_ts,
                  long long k_ts, long long v_ts, cudaStream_t s) {
  using C = FaCfg<D>;
  CUtensorMap tq, tk, tv;
  int rc;
  const uint64_t kv_rows = (uint64_t)(p.B - 1) * p.kv_brows + p.Sk;
  if ((rc = make_map_bf16(&tq, q, (uint64_t)p.hq * D, (uint64_t)p.B * p.Sq, (uint64_t)q_ts, 64, 128))) return rc;
  if ((rc = make_map_bf16(&tk, k, (uint64_t)p.hkv * D, kv_rows, (uint64_t)k_ts, 64, 128))) return rc;
  if ((rc = make_map_bf16(&tv, v, (uint64_t)p.hkv * D, kv_rows, (uint64_t)v_ts, 64, 128))) return rc;
  static bool attr = false;
  if (!attr) {
    cudaFuncSetAttribute(fa_fwd_tc_kernel<D>, cudaFuncAttributeMaxDynamicSharedMemorySize, C::SMEM);
    attr = true;
  }
  p.tiles_x = (p.Sq + 255) / 256;
  p.wait_ns = g_lb_flag_wait_ns;
  const long long grid = (long long)push.n_mov + (long long)p.tiles_x * p.hq * p.B;
  if (grid > 2147483647LL) return LB_ERR_SHAPE;
  fa_fwd_tc_kernel<D><<<(unsigned)grid, FA_FWD_THREADS, C::SMEM, s>>>(tq, tk, tv, p, push);
  LB_CHECK_LAUNCH();
  return LB_OK;
}

}  // namespace

// Copies the status words of the tcgen05 attention kernels to host memory and clears them.
extern "C" int lb_flash_status(void* out) {
  cudaError_t e = cudaMemcpyFromSymbol(out, g_fa_status, sizeof(unsigned int) * 4);
  if (e != cudaSuccess) { g_lb_last_cuda_error = (int)e; return LB_ERR_LAUNCH; }
  unsigned int zeros[4] = {0, 0, 0, 0};
  cudaMemcpyToSymbol(g_fa_status, zeros, sizeof(zeros));
  return LB_OK;
}

#ifdef LB_FA_PROFILE
extern "C" int lb_flash_prof(void* out) {
  cudaMemcpyFromSymbol(out, g_fa_prof, sizeof(unsigned long long) * 16);
  unsigned long long zeros[16] = {0};
  cudaMemcpyToSymbol(g_fa_prof, zeros, sizeof(zeros));
  return LB_OK;
}
#endif

// Same contract as lb_flash_fwd (flash_attn.cu); head_dim 64 or 128, all pointers 16-byte
// aligned, token strides multiples of 8, causal needs Sk >= Sq.  Returns LB_ERR_SHAPE otherwise.
extern "C" int lb_flash_fwd_tc(const void* q, const void* k, const void* v, void* o, void* lse, int B, int Sq, int Sk,
                               int hq, int hkv, int d, long long q_ts, long long k_ts, long long v_ts, long long o_ts,
                               float scale, int causal, void* stream) {
  if (B <= 0 || Sq <= 0 || Sk <= 0 || hq % hkv) return LB_ERR_SHAPE;
  if ((q_ts | k_ts | v_ts | o_ts) % 8) return LB_ERR_SHAPE;
  if (causal && Sk < Sq) return LB_ERR_SHAPE;
  if (((uintptr_t)q | (uintptr_t)k | (uintptr_t)v | (uintptr_t)o) & 15) return LB_ERR_ARG;
  FaFwdParams p{(bf16*)o, (float*)lse, B, Sq, Sk, hq, hkv, o_ts, scale, causal, Sk, nullptr, 0u, 0};
  FaPush push;
  memset(&push, 0, sizeof(push));
  cudaStream_t s = (cudaStream_t)stream;
  switch (d) {
    case 64: return launch_fa_fwd<64>(q, k, v, p, push, q_ts, k_ts, v_ts, s);
    case 128: return launch_fa_fwd<128>(q, k, v, p, push, q_ts, k_ts, v_ts, s);
    default: return LB_ERR_SHAPE;
  }
}

// Warps per CTA of the forward kernel: every mover warp adds 1 to a key block's arrival word for K
// and 1 for V, so a block is complete at (calls so far) * 2 * this.
extern "C" int lb_flash_fwd_cp_mover_warps() { return FA_FWD_THREADS / 32; }

// Context-parallel forward: attention of q [B, Sq, hq, d] over the first Sk keys of the gather
// buffers kg / vg ([B, S_full, hkv*d] contiguous, this rank's peer-visible buffers), each 128-key
// block gated on `flags` [B][S_full/128] reaching `flag_target`.  With n_mov > 0 the same launch
// also pushes this rank's two zig-zag chunks of k_src / v_src ([B, 2*chunk_rows, hkv, d]) into
// every rank's buffers (kdst / vdst / flag_ptrs: host arrays of n_ranks pointers).
// chunk_rows must be a multiple of 128; S_full = 2 * n_ranks * chunk_rows.
extern "C" int lb_flash_fwd_cp(const void* q, const void* kg, const void* vg, void* o, void* lse, int B, int Sq, int Sk,
                               int S_full, int hq, int hkv, int d, long long q_ts, long long o_ts, float scale,
                               int causal, const void* flags, unsigned int flag_target, int n_mov, const void* k_src,
                               const void* v_src, long long k_ts, long long v_ts, int n_ranks, int rank,
                               void* const* kdst, void* const* vdst, void* const* flag_ptrs, int chunk_rows,
                               void* stream) {
  if (B <= 0 || Sq <= 0 || Sk <= 0 || Sk > S_full || hq % hkv || (S_full % 128)) return LB_ERR_SHAPE;
  if ((q_ts | o_ts) % 8) return LB_ERR_SHAPE;
  if (causal && Sk < Sq) return LB_ERR_SHAPE;
  FaFwdParams p{(bf16*)o, (float*)lse, B, Sq, Sk, hq, hkv, o_ts, scale, causal, S_full, (const unsigned int*)flags,
                flag_target, 0};
  FaPush push;
  memset(&push, 0, sizeof(push));
  if (n_mov > 0) {
    if (n_ranks < 1 || n_ranks > FA_MAX_RANKS || (chunk_rows % 128) || S_full != 2 * n_ranks * chunk_rows) return LB_ERR_SHAPE;
    if ((k_ts | v_ts) % 8) return LB_ERR_SHAPE;
    push.n_mov = n_mov; push.n_ranks = n_ranks; push.rank = rank; push.chunk_rows = chunk_rows; push.row_elems = hkv * d;
    push.k_src = (const bf16*)k_src; push.v_src = (const bf16*)v_src; push.k_ts = k_ts; push.v_ts = v_ts;
    for (int r = 0; r < n_ranks; r++) {
      push.k_dst[r] = (bf16*)kdst[r]; push.v_dst[r] = (bf16*)vdst[r]; push.flags[r] = (unsigned int*)flag_ptrs[r];
    }
  }
  cudaStream_t s = (cudaStream_t)stream;
  const long long kts = (long long)hkv * d;
  switch (d) {
    case 64: return launch_fa_fwd<64>(q, kg, vg, p, push, q_ts, kts, kts, s);
    case 128: return launch_fa_fwd<128>(q, kg, vg, p, push, q_ts, kts, kts, s);
    default: return LB_ERR_SHAPE;
  }
}
