// FlashAttention backward on the 5th-generation tensor cores (sm_100a), head_dim 64 or 128.
//
// One CTA owns a block of 128 keys of one (batch, kv head) and walks over every 128-query block
// (of every query head of the GQA group) that can see it.  Per query block, five tcgen05 MMAs:
//     S   = Q K^T            [128 q x 128 k]   (K-major operands)
//     dP  = dO V^T           [128 q x 128 k]
//     dV += P^T dO           [128 k x d]       A = P as MN-major operand, B = dO MN-major
//     dK += dS^T Q           [128 k x d]       A = dS MN-major, B = Q MN-major
//     dQ  = dS K             [128 q x d]       A = dS K-major,  B = K MN-major
// S, dP, dQ, dV, dK live in TMEM (dV / dK accumulate there across the whole loop, so no
// rescaling is ever needed).  512 math threads (16 warps; thread = one query row x a quarter of
// the columns) read S and dP with tcgen05.ld, form P = exp(scale S - lse) and
// dS = P (dP - delta) scale in registers, and write both as bf16 into 128B-swizzled shared
// memory, where the same bytes serve as K-major (dQ) and MN-major (dV, dK) MMA operands.
// The gradient MMAs of a query block run in the order dQ, dV, dK: with head_dim 64 each dQ tile
// goes TMEM -> registers -> a per-warp staging area -> one asynchronous bulk reduce-add
// (cp.reduce.async.bulk .add.f32) per warp into an fp32 accumulator in global memory while dV and dK
// are still on the tensor pipe, so the drain (about 1200 cycles with its proxy fence) is off the
// critical path.  The accumulator's layout is the staging layout (un-permuted by the final convert
// kernel), so no atomic instructions pass through the load/store pipe.
// Warp roles (576 threads): warp 0 TMA producer, warp 1 MMA issuer + TMEM owner, warps 2-17 math.
// With head_dim 128 the dQ tile aliases the dP columns (TMEM is 512 columns), Q has two stages and
// dO one; with head_dim 64 Q and dO have three stages each and S/dP of the next query block are
// issued while the current one is still in the math warps.
// All waits are bounded; on expiry a status word is set and the CTA drains and frees its TMEM.
#include <stdlib.h>
#include "tcgen05.cuh"

static __device__ unsigned int g_fab_status[4] = {0, 0, 0, 0};
// Developer instrumentation (build with -DLB_FA_PROFILE): summed cycles per phase, see lb_flash_bwd_prof().
#ifdef LB_FA_PROFILE
static __device__ unsigned long long g_fab_prof[16];
#endif

namespace {
using namespace bw;

struct FaBwdParams {
  const bf16 *o, *dout;
  const float* lse;
  float *delta, *dq_acc;
  bf16 *dq, *dk, *dv;
  int B, Sq, Sk, hq, hkv;
  long long o_ts, do_ts, dq_ts, dk_ts, dv_ts;
  float scale;
  int causal;
  int kv_brows;   // rows between consecutive batches in the K/V tensor maps (>= Sk)
};

template <int D>
struct BwdCfg {
  static constexpr int BM = 128, BN = 128;
  // Q and dO go through separate stage rings.  head_dim 64: three stages each, so the loads of
  // query block i+1 are in flight while the gradient MMAs of block i-1 still read their stage
  // (with fewer stages the issuer was measured waiting 1450 cycles per block on TMA latency).
  // head_dim 128 (shared memory is short): one stage each; the gradient MMAs run in the order
  // dQ, dV, dK, so dO's stage is released while dK is still running.
  static constexpr int QS = (D == 64) ? 3 : 1;
  static constexpr int DS = (D == 64) ? 3 : 1;
  static constexpr bool EARLY = (D == 64);              // issue S/dP of block i+1 before dV/dK/dQ of block i
  static constexpr int ATOMS = D / 64;
  static constexpr int ATOM_BYTES = 128 * 128;
  static constexpr int TILE_BYTES = ATOMS * ATOM_BYTES;
  static constexpr int P_BYTES = 2 * ATOM_BYTES;
  static constexpr int DQC = D / 4;                     // dQ / dK / dV columns per math thread
  static constexpr int STG_WARP = 32 * DQC * 4;         // bytes of dQ staging per warp
  static constexpr int STG_BYTES = 16 * STG_WARP;       // 32 KiB (d = 64) or 64 KiB (d = 128)
  static constexpr bool STG_ALIAS = (D == 128);         // staging shares the P/dS bytes when smem is short
  static constexpr int OFF_K = 0;
  static constexpr int OFF_V = OFF_K + TILE_BYTES;
  static constexpr int OFF_Q = OFF_V + TILE_BYTES;              // [QS]
  static constexpr int OFF_DO = OFF_Q + QS * TILE_BYTES;        // [DS]
  static constexpr int OFF_P = OFF_DO + DS * TILE_BYTES;
  static constexpr int OFF_DS = OFF_P + P_BYTES;
  static constexpr int OFF_STG = STG_ALIAS ? OFF_P : OFF_DS + P_BYTES;
  static constexpr int OFF_BAR = STG_ALIAS ? OFF_DS + P_BYTES : OFF_STG + STG_BYTES;
  static constexpr int SMEM = OFF_BAR + 256 + 1024;
  static constexpr int NBAR = 1 + 2 * QS + 2 * DS + 7;
  static constexpr int NTHREADS = 576;
  // TMEM columns
  static constexpr int COL_S = 0, COL_DP = 128;
  static constexpr int COL_DQ = (D == 64) ? 256 : 128;          // aliases dP for d = 128
  static constexpr int COL_DV = (D == 64) ? 320 : 256;
  static constexpr int COL_DK = 384;
  // Swizzle of the 16-byte chunks of one thread's dQ row segment inside its warp's staging area
  // (keeps the 16-byte shared-memory stores of a warp conflict-free).
  __host__ __device__ static constexpr int stg_chunk(int c, int lane) {
    return (D == 64) ? (c ^ ((lane >> 1) & 3)) : (c ^ (lane & 7));
  }
};

// fp32 dQ accumulator layout: tile (b, h, mblock) -> 16 warp slots (part * 4 + quad) -> 32 lanes ->
// D/4 floats in swizzled 16-byte chunks.  Element (row r of the tile, column col):
//   quad = r / 32, lane = r % 32, part = col / (D/4), chunk = (col % (D/4)) / 4.
template <int D>
__global__ void fa_dq_convert_kernel(const FaBwdParams p) {
  using C = BwdCfg<D>;
  constexpr int VPR = D / 8;
  const int n_mblocks = (p.Sq + 127) / 128;
  const long long total = (long long)p.B * p.Sq * p.hq * VPR;
  for (long long idx = (long long)blockIdx.x * blockDim.x + threadIdx.x; idx < total;
       idx += (long long)gridDim.x * blockDim.x) {
    const int v = (int)(idx % VPR);
    const long long th = idx / VPR;
    const int h = (int)(th % p.hq);
    const long long bi = th / p.hq;
    const int b = (int)(bi / p.Sq), row = (int)(bi % p.Sq);
    const int mblock = row >> 7, r = row & 127, quad = r >> 5, lane = r & 31;
    const int col0 = v * 8, part = col0 / C::DQC, c0 = (col0 % C::DQC) >> 2;
    const float* tile = p.dq_acc + (((long long)b * p.hq + h) * n_mblocks + mblock) * (128 * D) +
                        (long long)(part * 4 + quad) * (32 * C::DQC) + lane * C::DQC;
    const float4 a = *reinterpret_cast<const float4*>(tile + C::stg_chunk(c0, lane) * 4);
    const float4 c = *reinterpret_cast<const float4*>(tile + C::stg_chunk(c0 + 1, lane) * 4);
    const float f[8] = {a.x, a.y, a.z, a.w, c.x, c.y, c.z, c.w};
    *reinterpret_cast<uint4*>(p.dq + bi * p.dq_ts + (long long)h * D + v * 8) = pack8(f);
  }
}

// delta[b, h, i] = sum_d o * do.  D/8 threads per (token, head), 16 bytes per thread per tensor.
template <int D>
__global__ void fa_delta_kernel(const FaBwdParams p) {
  constexpr int TPR = D / 8;                                   // threads per row: 8 or 16
  const long long total = (long long)p.B * p.Sq * p.hq;
  const int rpb = blockDim.x / TPR;                            // rows per block and iteration
  const int sub = threadIdx.x % TPR;
  // every thread of the block runs the same number of iterations, so the shuffles see whole warps
  for (long long base = (long long)blockIdx.x * rpb; base < total; base += (long long)gridDim.x * rpb) {
    const long long idx = base + threadIdx.x / TPR;
    const bool live = idx < total;
    float s = 0.f;
    int h = 0;
    long long bi = 0;
    if (live) {
      h = (int)(idx % p.hq);
      bi = idx / p.hq;
      float a[8], e[8];
      unpack8(*reinterpret_cast<const uint4*>(p.o + bi * p.o_ts + (long long)h * D + sub * 8), a);
      unpack8(*reinterpret_cast<const uint4*>(p.dout + bi * p.do_ts + (long long)h * D + sub * 8), e);
#pragma unroll
      for (int k = 0; k < 8; k++) s += a[k] * e[k];
    }
#pragma unroll
    for (int o = TPR / 2; o > 0; o >>= 1) s += __shfl_xor_sync(0xffffffffu, s, o);   // whole warps stay converged
    if (live && sub == 0) {
      const int b = (int)(bi / p.Sq), i = (int)(bi % p.Sq);
      p.delta[((long long)b * p.hq + h) * p.Sq + i] = s;
    }
  }
}

template <int D>
__global__ void __launch_bounds__(576, 1)
fa_bwd_tc_kernel(const __grid_constant__ CUtensorMap tq, const __grid_constant__ CUtensorMap tk,
                 const __grid_constant__ CUtensorMap tv, const __grid_constant__ CUtensorMap tdo, const FaBwdParams p) {
  using C = BwdCfg<D>;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~(uintptr_t)1023);
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + C::OFF_BAR);
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + C::NBAR);
  __shared__ int s_abort[2];     // {abort, extra wait in ms}: see bw::mbar_wait

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const uint32_t sbase = smem_u32(smem);
  const uint32_t bar0 = smem_u32(bars);
  const uint32_t kv_full = bar0;
  auto q_full = [&](int s) { return bar0 + 8u * (1 + s); };
  auto q_empty = [&](int s) { return bar0 + 8u * (1 + C::QS + s); };
  auto do_full = [&](int s) { return bar0 + 8u * (1 + 2 * C::QS + s); };
  auto do_empty = [&](int s) { return bar0 + 8u * (1 + 2 * C::QS + C::DS + s); };
  const uint32_t bar1 = bar0 + 8u * (1 + 2 * C::QS + 2 * C::DS);
  const uint32_t sdp_full = bar1, sdp_free = bar1 + 8, pds_full = bar1 + 16, dq_full = bar1 + 24, dq_free = bar1 + 32,
                 pds_free = bar1 + 40, stg_free = bar1 + 48;

  const int nblk = blockIdx.x, hk = blockIdx.y, b = blockIdx.z;
  const int n0 = nblk * C::BN;
  const int off = p.Sk - p.Sq;
  const int rep = p.hq / p.hkv;
  const int n_mblocks = (p.Sq + C::BM - 1) / C::BM;
  int mb_first = 0;
  if (p.causal) {
    const int first_row = n0 - off;
    mb_first = first_row > 0 ? first_row / C::BM : 0;
  }
  const int per_head = n_mblocks > mb_first ? n_mblocks - mb_first : 0;
  const int total_it = per_head * rep;

  if (threadIdx.x == 0) {
    s_abort[0] = 0;
    s_abort[1] = 0;
    mbar_init(kv_full, 1);
    for (int s = 0; s < C::QS; s++) { mbar_init(q_full(s), 1); mbar_init(q_empty(s), 1); }
    for (int s = 0; s < C::DS; s++) { mbar_init(do_full(s), 1); mbar_init(do_empty(s), 1); }
    mbar_init(sdp_full, 1);
    mbar_init(sdp_free, 512);
    mbar_init(pds_full, 512);
    mbar_init(dq_full, 1);
    mbar_init(dq_free, 512);
    mbar_init(pds_free, 1);
    mbar_init(stg_free, 16);
    mbar_init_fence();
    prefetch_tmap(&tq); prefetch_tmap(&tk); prefetch_tmap(&tv); prefetch_tmap(&tdo);
  }
  if (warp == 1) tmem_alloc(smem_u32(tmem_slot), 512);
  fence_before();
  __syncthreads();
  fence_after();
  const uint32_t tmem_base = *tmem_slot;
  volatile int* abort_flag = s_abort;

  if (warp == 0) {
    // ------------------------------- TMA producer -------------------------------
    if (lane == 0 && total_it > 0) {
      mbar_expect_tx(kv_full, 2 * C::TILE_BYTES);
#pragma unroll
      for (int a = 0; a < C::ATOMS; a++) {
        tma_load_2d(sbase + C::OFF_K + a * C::ATOM_BYTES, &tk, hk * D + a * 64, b * p.kv_brows + n0, kv_full);
        tma_load_2d(sbase + C::OFF_V + a * C::ATOM_BYTES, &tv, hk * D + a * 64, b * p.kv_brows + n0, kv_full);
      }
      bool ok = true;
      for (int it = 0; it < total_it; it++) {
        const int qs = it % C::QS, ds = it % C::DS;
        const int h = hk * rep + it / per_head;
        const int m0 = (mb_first + it % per_head) * C::BM;
        if (!mbar_wait(q_empty(qs), (((uint32_t)(it / C::QS)) & 1u) ^ 1u, abort_flag)) { ok = false; break; }
        mbar_expect_tx(q_full(qs), C::TILE_BYTES);
#pragma unroll
        for (int a = 0; a < C::ATOMS; a++)
          tma_load_2d(sbase + C::OFF_Q + qs * C::TILE_BYTES + a * C::ATOM_BYTES, &tq, h * D + a * 64, b * p.Sq + m0, q_full(qs));
        if (!mbar_wait(do_empty(ds), (((uint32_t)(it / C::DS)) & 1u) ^ 1u, abort_flag)) { ok = false; break; }
        mbar_expect_tx(do_full(ds), C::TILE_BYTES);
#pragma unroll
        for (int a = 0; a < C::ATOMS; a++)
          tma_load_2d(sbase + C::OFF_DO + ds * C::TILE_BYTES + a * C::ATOM_BYTES, &tdo, h * D + a * 64, b * p.Sq + m0, do_full(ds));
      }
      if (!ok) atomicExch(&g_fab_status[0], 1u);
    }
  } else if (warp == 1) {
    // ------------------------------- MMA issuer -------------------------------
    if (lane == 0 && total_it > 0) {
      const uint32_t idesc_s = make_idesc(128, 128, 0, 0);     // S, dP: K-major A and B
      const uint32_t idesc_kv = make_idesc(128, D, 1, 1);      // dV, dK: MN-major A and B
      const uint32_t idesc_dq = make_idesc(128, D, 0, 1);      // dQ: K-major A, MN-major B
      // descriptor bases; a stage / k-step only changes the 16-byte-granular start address
      const uint64_t kK = make_desc(sbase + C::OFF_K, 16, 1024), kV = make_desc(sbase + C::OFF_V, 16, 1024);
      const uint64_t kQ = make_desc(sbase + C::OFF_Q, 16, 1024), kDO = make_desc(sbase + C::OFF_DO, 16, 1024);
      const uint64_t kDS = make_desc(sbase + C::OFF_DS, 16, 1024);
      const uint64_t mK = make_desc(sbase + C::OFF_K, C::ATOM_BYTES, 1024);
      const uint64_t mQ = make_desc(sbase + C::OFF_Q, C::ATOM_BYTES, 1024), mDO = make_desc(sbase + C::OFF_DO, C::ATOM_BYTES, 1024);
      const uint64_t mP = make_desc(sbase + C::OFF_P, C::ATOM_BYTES, 1024), mDS = make_desc(sbase + C::OFF_DS, C::ATOM_BYTES, 1024);
      // S and dP of query block `it`: needs its Q / dO stages and the S / dP columns (held by the
      // math warps until they have block it-1 in registers; with head_dim 128 dQ of block it-1
      // sits in the dP columns until it has been drained)
      auto issue_s_dp = [&](int it) -> bool {
        const int qs = it % C::QS, ds = it % C::DS;
        if (!mbar_wait(q_full(qs), ((uint32_t)(it / C::QS)) & 1u, abort_flag)) return false;
        if (!mbar_wait(do_full(ds), ((uint32_t)(it / C::DS)) & 1u, abort_flag)) return false;
        if (it > 0 && !mbar_wait(C::EARLY ? sdp_free : dq_free, (uint32_t)(it - 1) & 1u, abort_flag)) return false;
        fence_after();
        const uint64_t qo = (uint64_t)((qs * C::TILE_BYTES) >> 4), go = (uint64_t)((ds * C::TILE_BYTES) >> 4);
#pragma unroll
        for (int s = 0; s < D / 16; s++) {
          const uint64_t o = (uint64_t)(((s >> 2) * C::ATOM_BYTES + (s & 3) * 32) >> 4);
          umma_bf16(tmem_base + C::COL_S, kQ + qo + o, kK + o, idesc_s, s ? 1u : 0u);
        }
#pragma unroll
        for (int s = 0; s < D / 16; s++) {
          const uint64_t o = (uint64_t)(((s >> 2) * C::ATOM_BYTES + (s & 3) * 32) >> 4);
          umma_bf16(tmem_base + C::COL_DP, kDO + go + o, kV + o, idesc_s, s ? 1u : 0u);
        }
        umma_commit(sdp_full);
        return true;
      };
      // dQ first: its tile can leave for global memory while dV and dK are still on the tensor
      // pipe.  dV releases the dO stage, dK the Q stage and the P / dS bytes.
      auto issue_grads = [&](int it) -> bool {
        const int qs = it % C::QS, ds = it % C::DS;
        if (!mbar_wait(pds_full, (uint32_t)it & 1u, abort_flag)) return false;
        if (C::EARLY && it > 0 && !mbar_wait(dq_free, (uint32_t)(it - 1) & 1u, abort_flag)) return false;
        fence_after();
        const uint64_t qo = (uint64_t)((qs * C::TILE_BYTES) >> 4), go = (uint64_t)((ds * C::TILE_BYTES) >> 4);
        const uint32_t acc0 = it ? 1u : 0u;
#pragma unroll
        for (int s = 0; s < C::BN / 16; s++)                                   // dQ = dS K      (K = 128 keys)
          umma_bf16(tmem_base + C::COL_DQ, kDS + (uint64_t)(((s >> 2) * C::ATOM_BYTES + (s & 3) * 32) >> 4),
                    mK + (uint64_t)(s * 128), idesc_dq, s ? 1u : 0u);
        umma_commit(dq_full);
        umma_bf16(tmem_base + C::COL_DV, mP, mDO + go, idesc_kv, acc0);       // dV += P^T dO   (K = 128 queries)
#pragma unroll
        for (int s = 1; s < C::BM / 16; s++)
          umma_bf16(tmem_base + C::COL_DV, mP + (uint64_t)(s * 128), mDO + go + (uint64_t)(s * 128), idesc_kv, 1u);
        umma_commit(do_empty(ds));
        umma_bf16(tmem_base + C::COL_DK, mDS, mQ + qo, idesc_kv, acc0);       // dK += dS^T Q
#pragma unroll
        for (int s = 1; s < C::BM / 16; s++)
          umma_bf16(tmem_base + C::COL_DK, mDS + (uint64_t)(s * 128), mQ + qo + (uint64_t)(s * 128), idesc_kv, 1u);
        umma_commit(q_empty(qs));
        umma_commit(pds_free);
        return true;
      };
      bool ok = mbar_wait(kv_full, 0, abort_flag);
      if (ok) ok = issue_s_dp(0);
      for (int it = 0; it < total_it && ok; it++) {
        if (C::EARLY && it + 1 < total_it) ok = issue_s_dp(it + 1);
        if (ok) ok = issue_grads(it);
        if (!C::EARLY && ok && it + 1 < total_it) ok = issue_s_dp(it + 1);
      }
      if (!ok) atomicExch(&g_fab_status[0], 2u);
    }
  } else {
    // ------------------------------- math warps -------------------------------
    const int quad = warp & 3;
    const int part = (warp - 2) >> 2;               // which 32 of the 128 key columns / which quarter of d
    const int rit = quad * 32 + lane;               // row inside the 128-row tile
    const uint32_t lane_addr = tmem_base + ((uint32_t)(quad * 32) << 16);
    const float sl2 = p.scale * 1.4426950408889634f;
    const float l2e = 1.4426950408889634f;
    uint8_t* sProw = smem + C::OFF_P + (part >> 1) * C::ATOM_BYTES;
    uint8_t* sDSrow = smem + C::OFF_DS + (part >> 1) * C::ATOM_BYTES;
    constexpr int DQC = C::DQC;
    bool ok = true;
    int prev_m0 = 0, prev_h = 0;
    const int ws = part * 4 + quad;                 // this warp's slot in the dQ staging / accumulator layout
    uint8_t* stg = smem + C::OFF_STG + ws * C::STG_WARP;
    const int n_mblocks_acc = n_mblocks;
    int n_flushed = 0;
    // dQ of query block `it_prev`: TMEM -> registers -> this warp's staging area -> one asynchronous
    // bulk reduce-add into the fp32 accumulator (whose layout is the staging layout).  Reduce-adds
    // issued from registers (red.global.add.v4.f32) were measured slower: the warps stall on the
    // load/store pipe, while the bulk engine drains in the background.
    auto flush_dq = [&](int it_prev) -> bool {
      if (!mbar_wait(dq_full, (uint32_t)it_prev & 1u, abort_flag)) return false;
      fence_after();
      uint32_t r[DQC];
      tmem_ld<DQC>(lane_addr + C::COL_DQ + part * DQC, r);
      tmem_ld_wait();
      fence_before();
      mbar_arrive(dq_free);
      if (C::STG_ALIAS) {
        // the staging bytes are the P / dS bytes: dV and dK must have finished reading them
        if (!mbar_wait(pds_free, (uint32_t)it_prev & 1u, abort_flag)) return false;
      } else {
        if (lane == 0) bulk_wait_read();            // this warp's previous bulk op has read the staging area
        __syncwarp();
      }
#pragma unroll
      for (int c = 0; c < DQC / 4; c++)
        *reinterpret_cast<uint4*>(stg + lane * (DQC * 4) + C::stg_chunk(c, lane) * 16) =
            make_uint4(r[c * 4], r[c * 4 + 1], r[c * 4 + 2], r[c * 4 + 3]);
      fence_proxy_async_smem();
      __syncwarp();
      if (lane == 0) {
        float* dst = p.dq_acc + (((long long)b * p.hq + prev_h) * n_mblocks_acc + (prev_m0 >> 7)) * (128 * D) +
                     (long long)ws * (32 * DQC);
        bulk_reduce_add_f32(dst, smem_u32(stg), C::STG_WARP);
        bulk_commit();
        if (C::STG_ALIAS) {                          // the bytes are P/dS again in the next block
          bulk_wait_read();
          mbar_arrive(stg_free);
        }
      }
      n_flushed++;
      return true;
    };
    for (int it = 0; it < total_it; it++) {
      const int h = hk * rep + it / per_head;
      const int m0 = (mb_first + it % per_head) * C::BM;
      const int row = m0 + rit;
      float lse_r = INFINITY, delta_r = 0.f;
      if (row < p.Sq) {
        const long long li = ((long long)b * p.hq + h) * p.Sq + row;
        lse_r = p.lse[li];
        delta_r = p.delta[li];
      }
      if (!mbar_wait(sdp_full, (uint32_t)it & 1u, abort_flag)) { ok = false; break; }
      fence_after();
      uint32_t sr[32], dr[32];
      tmem_ld32(lane_addr + C::COL_S + part * 32, sr);
      tmem_ld32(lane_addr + C::COL_DP + part * 32, dr);
      tmem_ld_wait();
      fence_before();
      mbar_arrive(sdp_free);
      // P and dS for this thread's 32 keys
      const int key0 = n0 + part * 32;
      const bool need_mask = (n0 + C::BN > p.Sk) || (p.causal && (n0 + C::BN - 1 > m0 + quad * 32 + off));
      const int lim = (p.causal ? min(p.Sk - 1, row + off) : p.Sk - 1) - key0;
      const float nl = -lse_r * l2e;
      const float nds = -delta_r * p.scale;
      uint32_t pp[16], dd[16];
#pragma unroll
      for (int i = 0; i < 32; i += 2) {
        float p0 = exp2f(fmaf(__uint_as_float(sr[i]), sl2, nl));
        float p1 = exp2f(fmaf(__uint_as_float(sr[i + 1]), sl2, nl));
        if (need_mask) {
          if (i > lim) p0 = 0.f;
          if (i + 1 > lim) p1 = 0.f;
        }
        const float d0 = p0 * fmaf(__uint_as_float(dr[i]), p.scale, nds);
        const float d1 = p1 * fmaf(__uint_as_float(dr[i + 1]), p.scale, nds);
        bf162 pb = __floats2bfloat162_rn(p0, p1), db = __floats2bfloat162_rn(d0, d1);
        pp[i >> 1] = *reinterpret_cast<uint32_t*>(&pb);
        dd[i >> 1] = *reinterpret_cast<uint32_t*>(&db);
      }
      if (C::EARLY && it > 0) {
        if (!flush_dq(it - 1)) { ok = false; break; }
      }
      // P / dS bytes may be rewritten once dV, dK and dQ of the previous block have read them
      // (and, where the dQ staging shares them, once every warp's bulk op has read its staging)
      if (it > 0 && !mbar_wait(pds_free, (uint32_t)(it - 1) & 1u, abort_flag)) { ok = false; break; }
      if (C::STG_ALIAS && it > 0 && !mbar_wait(stg_free, (uint32_t)(it - 1) & 1u, abort_flag)) { ok = false; break; }
#pragma unroll
      for (int c = 0; c < 4; c++) {
        const uint32_t o = sw128_off(rit, (part & 1) * 4 + c);
        *reinterpret_cast<uint4*>(sProw + o) = make_uint4(pp[c * 4], pp[c * 4 + 1], pp[c * 4 + 2], pp[c * 4 + 3]);
        *reinterpret_cast<uint4*>(sDSrow + o) = make_uint4(dd[c * 4], dd[c * 4 + 1], dd[c * 4 + 2], dd[c * 4 + 3]);
      }
      fence_proxy_async_smem();
      mbar_arrive(pds_full);
      prev_m0 = m0;
      prev_h = h;
      if (!C::EARLY) {   // dQ aliases dP: it must be drained before the next S/dP can be issued
        if (!flush_dq(it)) { ok = false; break; }
      }
    }
    if (C::EARLY && ok && total_it > 0) ok = flush_dq(total_it - 1);
    if (lane == 0 && n_flushed > 0) bulk_wait_read();   // staging must outlive the last bulk read
    if (ok && total_it > 0) ok = mbar_wait(pds_free, (uint32_t)(total_it - 1) & 1u, abort_flag);   // every MMA has finished
    if (ok && total_it > 0) {
      fence_after();
      const int key = n0 + rit;
      bf16* dkrow = p.dk + ((long long)b * p.Sk + key) * p.dk_ts + (long long)hk * D + part * DQC;
      bf16* dvrow = p.dv + ((long long)b * p.Sk + key) * p.dv_ts + (long long)hk * D + part * DQC;
      uint32_t r[DQC];
      float f[DQC];
      tmem_ld<DQC>(lane_addr + C::COL_DK + part * DQC, r);
      tmem_ld_wait();
      if (key < p.Sk) {
#pragma unroll
        for (int i = 0; i < DQC; i++) f[i] = __uint_as_float(r[i]);
#pragma unroll
        for (int g = 0; g < DQC / 8; g++) *reinterpret_cast<uint4*>(dkrow + g * 8) = pack8(f + g * 8);
      }
      tmem_ld<DQC>(lane_addr + C::COL_DV + part * DQC, r);
      tmem_ld_wait();
      if (key < p.Sk) {
#pragma unroll
        for (int i = 0; i < DQC; i++) f[i] = __uint_as_float(r[i]);
#pragma unroll
        for (int g = 0; g < DQC / 8; g++) *reinterpret_cast<uint4*>(dvrow + g * 8) = pack8(f + g * 8);
      }
    } else if (total_it == 0) {
      // no query sees these keys: their gradients are zero
      const int key = n0 + rit;
      if (key < p.Sk) {
        bf16* dkrow = p.dk + ((long long)b * p.Sk + key) * p.dk_ts + (long long)hk * D + part * DQC;
        bf16* dvrow = p.dv + ((long long)b * p.Sk + key) * p.dv_ts + (long long)hk * D + part * DQC;
        for (int c = 0; c < DQC / 8; c++) {
          *reinterpret_cast<uint4*>(dkrow + c * 8) = make_uint4(0, 0, 0, 0);
          *reinterpret_cast<uint4*>(dvrow + c * 8) = make_uint4(0, 0, 0, 0);
        }
      }
    }
    if (!ok && lane == 0) atomicExch(&g_fab_status[0], 3u);
  }

  fence_before();
  __syncthreads();
  if (warp == 1) {
    fence_after();
    tmem_dealloc(tmem_base, 512);
  }
}

template <int D>
int launch_fa_bwd(const void* q, const void* k, const void* v, const FaBwdParams& p, long long q_ts, long long k_ts,
                  long long v_ts, cudaStream_t s) {
  using C = BwdCfg<D>;
  CUtensorMap tq, tk, tv, tdo;
  int rc;
  if ((rc = make_map_bf16(&tq, q, (uint64_t)p.hq * D, (uint64_t)p.B * p.Sq, (uint64_t)q_ts, 64, 128))) return rc;
  const uint64_t kv_rows = (uint64_t)(p.B - 1) * p.kv_brows + p.Sk;
  if ((rc = make_map_bf16(&tk, k, (uint64_t)p.hkv * D, kv_rows, (uint64_t)k_ts, 64, 128))) return rc;
  if ((rc = make_map_bf16(&tv, v, (uint64_t)p.hkv * D, kv_rows, (uint64_t)v_ts, 64, 128))) return rc;
  if ((rc = make_map_bf16(&tdo, p.dout, (uint64_t)p.hq * D, (uint64_t)p.B * p.Sq, (uint64_t)p.do_ts, 64, 128))) return rc;
  static bool attr = false;
  if (!attr) {
    cudaFuncSetAttribute(fa_bwd_tc_kernel<D>, cudaFuncAttributeMaxDynamicSharedMemorySize, C::SMEM);
    attr = true;
  }
  const long long rows = (long long)p.B * p.Sq * p.hq;
  const long long rows_per_block = 256 / (D / 8);
  int dblocks = (int)((rows + rows_per_block - 1) / rows_per_block > lb_num_sms() * 16 ? lb_num_sms() * 16 : (rows + rows_per_block - 1) / rows_per_block);
  fa_delta_kernel<D><<<dblocks, 256, 0, s>>>(p);
  LB_CHECK_LAUNCH();
  dim3 grid((p.Sk + 127) / 128, p.hkv, p.B);
  fa_bwd_tc_kernel<D><<<grid, C::NTHREADS, C::SMEM, s>>>(tq, tk, tv, tdo, p);
  LB_CHECK_LAUNCH();
  const long long total = rows * (D / 8);
  int cblocks = (int)((total + 255) / 256 > lb_num_sms() * 16 ? lb_num_sms() * 16 : (total + 255) / 256);
  fa_dq_convert_kernel<D><<<cblocks, 256, 0, s>>>(p);
  LB_CHECK_LAUNCH();
  return LB_OK;
}

}  // namespace

// Copies the status words of the tcgen05 attention backward kernel to host memory and clears them.
extern "C" int lb_flash_bwd_status(void* out) {
  cudaError_t e = cudaMemcpyFromSymbol(out, g_fab_status, sizeof(unsigned int) * 4);
  if (e != cudaSuccess) { g_lb_last_cuda_error = (int)e; return LB_ERR_LAUNCH; }
  unsigned int zeros[4] = {0, 0, 0, 0};
  cudaMemcpyToSymbol(g_fab_status, zeros, sizeof(zeros));
  return LB_OK;
}

#ifdef LB_FA_PROFILE
extern "C" int lb_flash_bwd_prof(void* out) {
  cudaMemcpyFromSymbol(out, g_fab_prof, sizeof(unsigned long long) * 16);
  unsigned long long zeros[16] = {0};
  cudaMemcpyToSymbol(g_fab_prof, zeros, sizeof(zeros));
  return LB_OK;
}
#endif

// Same contract as lb_flash_bwd (flash_attn.cu) except for the scratch: dq_acc is zero-initialised
// fp32 of B * hq * ceil(Sq/128) * 128 * d elements (tile-permuted layout, see fa_dq_convert_kernel);
// delta is fp32 scratch [B, hq, Sq].  head_dim 64 or 128; causal needs Sk >= Sq.
static int flash_bwd_tc_impl(int kv_brows, const void* q, const void* k, const void* v, const void* o, const void* dout,
                               const void* lse, void* delta, void* dq_acc, void* dq, void* dk, void* dv, int B, int Sq,
                               int Sk, int hq, int hkv, int d, long long q_ts, long long k_ts, long long v_ts,
                               long long o_ts, long long do_ts, long long dq_ts, long long dk_ts, long long dv_ts,
                               float scale, int causal, void* stream) {
  if (B <= 0 || Sq <= 0 || Sk <= 0 || hq % hkv) return LB_ERR_SHAPE;
  if ((q_ts | k_ts | v_ts | o_ts | do_ts | dq_ts | dk_ts | dv_ts) % 8) return LB_ERR_SHAPE;
  if (causal && Sk < Sq) return LB_ERR_SHAPE;
  if (((uintptr_t)q | (uintptr_t)k | (uintptr_t)v | (uintptr_t)dout | (uintptr_t)dq | (uintptr_t)dk | (uintptr_t)dv) & 15)
    return LB_ERR_ARG;
  FaBwdParams p{(const bf16*)o, (const bf16*)dout, (const float*)lse, (float*)delta, (float*)dq_acc,
                (bf16*)dq, (bf16*)dk, (bf16*)dv, B, Sq, Sk, hq, hkv, o_ts, do_ts, dq_ts, dk_ts, dv_ts, scale, causal,
                kv_brows};
  cudaStream_t s = (cudaStream_t)stream;
  switch (d) {
    case 64: return launch_fa_bwd<64>(q, k, v, p, q_ts, k_ts, v_ts, s);
    case 128: return launch_fa_bwd<128>(q, k, v, p, q_ts, k_ts, v_ts, s);
    default: return LB_ERR_SHAPE;
  }
}

extern "C" int lb_flash_bwd_tc(const void* q, const void* k, const void* v, const void* o, const void* dout,
                               const void* lse, void* delta, void* dq_acc, void* dq, void* dk, void* dv, int B, int Sq,
                               int Sk, int hq, int hkv, int d, long long q_ts, long long k_ts, long long v_ts,
                               long long o_ts, long long do_ts, long long dq_ts, long long dk_ts, long long dv_ts,
                               float scale, int causal, void* stream) {
  return flash_bwd_tc_impl(Sk, q, k, v, o, dout, lse, delta, dq_acc, dq, dk, dv, B, Sq, Sk, hq, hkv, d, q_ts, k_ts, v_ts,
                           o_ts, do_ts, dq_ts, dk_ts, dv_ts, scale, causal, stream);
}

// Same, for K/V that are the first Sk rows of every batch of a longer buffer (kv_brows rows per
// batch): the context-parallel gather buffers.  dk / dv stay [B, Sk, hkv, d].
extern "C" int lb_flash_bwd_cp(const void* q, const void* k, const void* v, const void* o, const void* dout,
                               const void* lse, void* delta, void* dq_acc, void* dq, void* dk, void* dv, int B, int Sq,
                               int Sk, int kv_brows, int hq, int hkv, int d, long long q_ts, long long k_ts,
                               long long v_ts, long long o_ts, long long do_ts, long long dq_ts, long long dk_ts,
                               long long dv_ts, float scale, int causal, void* stream) {
  if (kv_brows < Sk) return LB_ERR_SHAPE;
  return flash_bwd_tc_impl(kv_brows, q, k, v, o, dout, lse, delta, dq_acc, dq, dk, dv, B, Sq, Sk, hq, hkv, d, q_ts, k_ts,
                           v_ts, o_ts, do_ts, dq_ts, dk_ts, dv_ts, scale, causal, stream);
}
