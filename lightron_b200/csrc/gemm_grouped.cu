// Grouped bf16 GEMM for sm_100a: up to 8 independent problems  C_i[M_i,N_i] (+)= op(A_i) op(B_i)^T
// in ONE persistent launch.
//
// Why: a single GEMM whose tile count is not a multiple of the SM count leaves SMs idle in its
// last wave (a weight gradient [2560, 2048] has 160 tiles for 148 SMs: the second wave is 8 %
// full).  Launching the data gradient and the weight gradient of a linear layer together, or
// the GEMMs of all local experts of a MoE layer, gives the scheduler short tiles to fill those
// holes.  The host computes a static schedule (longest tiles first, each to the least loaded
// CTA), uploads it once per shape, and every role of a CTA walks the same list, so no
// intra-kernel tile broadcast is needed.
//
// The main loop is the one of gemm_tcgen05.cu: TMA (128-byte swizzle, no multicast) -> 4-stage
// mbarrier ring -> tcgen05.mma 128x256x16 -> two 256-column TMEM accumulators -> tcgen05.ld
// epilogue overlapped with the next tile.  `accumulate` adds the old contents of C in the
// epilogue (gradient accumulation over micro-batches without a separate add).
// Every wait is bounded; on expiry the kernel records a status code (lb_gemm_grouped_status),
// stops issuing work, frees its TMEM and returns.
#include <cuda.h>
#include <string.h>
#include <algorithm>
#include <map>
#include <mutex>
#include <queue>
#include <vector>
#include "common.cuh"
#include "tcgen05.cuh"
#include "comm.cuh"

static __device__ unsigned int g_grp_status[4] = {0, 0, 0, 0};

namespace {

constexpr int BM = 128, BN = 256, BK = 64;
constexpr int STAGES = 4;
constexpr int A_BYTES = BM * BK * 2;
constexpr int B_BYTES = BN * BK * 2;
constexpr int STAGE_BYTES = A_BYTES + B_BYTES;
constexpr int SMEM_BYTES = STAGES * STAGE_BYTES + 1024 + 256;
constexpr int NUM_THREADS = 192;
constexpr int GROUP_M = 8;
constexpr int MAX_PROBLEMS = 8;

// epi selects the epilogue of a problem:
//   0  C = acc (+ C when accumulate)
//   1  SwiGLU forward: B is a fused [2 * half, K] gate | up weight.  Tile tn holds 128 gate columns
//      (accumulator columns 0..127) and the 128 up columns of the same index (128..255): both go to
//      C [M, 2 * half] as usual (the backward needs them) and silu(g) * u goes to C2 [M, half].
//   2  SwiGLU backward: acc is dh [M, half] of the down projection; the epilogue reads g | u from
//      C2 [M, 2 * half] and writes dg | du to C [M, 2 * half]; dh itself is never stored.
struct Problem {
  bf16* C;
  long long ldc;
  bf16* C2;
  long long ldc2;
  int M, N, K;
  int a_mn, b_mn, accumulate;
  int tiles_m, tiles_n, num_kb;
  int epi, half;
};

struct GroupedParams {
  CUtensorMap ta[MAX_PROBLEMS];
  CUtensorMap tb[MAX_PROBLEMS];
  Problem prob[MAX_PROBLEMS];
  const int* offsets;   // [grid + 1] first item of every CTA
  const int* items;     // (problem << 24) | tile index inside the problem
};

__device__ __forceinline__ void tile_coords(int t, const Problem& p, int& tm, int& tn) {
  const int group_size = GROUP_M * p.tiles_n;
  const int group = t / group_size;
  const int first_m = group * GROUP_M;
  const int gsz = min(p.tiles_m - first_m, GROUP_M);
  const int in_group = t - group * group_size;
  tm = first_m + in_group % gsz;
  tn = in_group / gsz;
}

__device__ __forceinline__ void give_up(volatile int* abort_flag, unsigned where) {
  *abort_flag = 1;
  atomicExch(&g_grp_status[0], 1u);
  atomicExch(&g_grp_status[1], where);
}

// One tile of the producer / of the MMA issuer, specialised on the operand majors: with the majors
// as compile-time constants every descriptor field and the number of TMA boxes is a constant (with
// run-time majors the producer issued predicated-off TMA instructions for the branch not taken and
// the tensor pipe lost a fifth of its activity), although the tile itself comes from a list in memory.
template <bool A_MN, bool B_MN>
__device__ __forceinline__ bool produce_tile(const CUtensorMap* ta, const CUtensorMap* tb, int m0, int n0, int num_kb,
                                             uint32_t smem_base, uint32_t bar_base, int& stage, uint32_t& phase,
                                             volatile int* abort_flag, int k_base = 0, int b_split = 0) {
  for (int kb = 0; kb < num_kb; kb++) {
    if (!bw::mbar_wait(bar_base + 8u * (STAGES + stage), phase ^ 1u, abort_flag)) return false;
    const uint32_t fb = bar_base + 8u * stage;
    bw::mbar_expect_tx(fb, STAGE_BYTES);
    const uint32_t sa = smem_base + stage * STAGE_BYTES;
    const uint32_t sb = sa + A_BYTES;
    const int k0 = k_base + kb * BK;
    if (!A_MN) {
      bw::tma_load_2d(sa, ta, k0, m0, fb);                                                      // box {64 k, 128 m}
    } else {
#pragma unroll
      for (int j = 0; j < BM / 64; j++) bw::tma_load_2d(sa + j * 8192, ta, m0 + 64 * j, k0, fb);  // box {64 m, 64 k}
    }
    if (!B_MN) {
      if (b_split > 0) {                       // two boxes {64 k, 128 n}: rows n0.. and b_split + n0.. of B
        bw::tma_load_2d(sb, tb, k0, n0, fb);
        bw::tma_load_2d(sb + (BN / 2) * BK * 2, tb, k0, b_split + n0, fb);
      } else {
        bw::tma_load_2d(sb, tb, k0, n0, fb);                                                    // box {64 k, 256 n}
      }
    } else {
#pragma unroll
      for (int j = 0; j < BN / 64; j++) bw::tma_load_2d(sb + j * 8192, tb, n0 + 64 * j, k0, fb);  // box {64 n, 64 k}
    }
    if (++stage == STAGES) { stage = 0; phase ^= 1u; }
  }
  return true;
}

template <bool A_MN, bool B_MN>
__device__ __forceinline__ bool mma_tile(uint32_t d_tmem, int num_kb, uint32_t smem_base, uint32_t bar_base, int& stage,
                                         uint32_t& phase, volatile int* abort_flag) {
  constexpr uint32_t idesc = (1u << 4) | (1u << 7) | (1u << 10) | ((A_MN ? 1u : 0u) << 15) | ((B_MN ? 1u : 0u) << 16) |
                             ((uint32_t)(BN >> 3) << 17) | ((uint32_t)(BM >> 4) << 24);
  constexpr uint32_t a_lbo = A_MN ? 8192u : 16u, b_lbo = B_MN ? 8192u : 16u;
  constexpr uint32_t a_kstep = A_MN ? 2048u : 32u, b_kstep = B_MN ? 2048u : 32u;   // bytes per K=16 slice
  for (int kb = 0; kb < num_kb; kb++) {
    if (!bw::mbar_wait(bar_base + 8u * stage, phase, abort_flag)) return false;
    bw::fence_after();
    const uint32_t sa = smem_base + stage * STAGE_BYTES;
    const uint32_t sb = sa + A_BYTES;
#pragma unroll
    for (int k = 0; k < BK / 16; k++) {
      const uint64_t ad = bw::make_desc(sa + k * a_kstep, a_lbo, 1024u);
      const uint64_t bd = bw::make_desc(sb + k * b_kstep, b_lbo, 1024u);
      bw::umma_bf16(d_tmem, ad, bd, idesc, (kb | k) ? 1u : 0u);
    }
    bw::umma_commit(bar_base + 8u * (STAGES + stage));   // frees this smem stage when the MMAs have read it
    if (++stage == STAGES) { stage = 0; phase ^= 1u; }
  }
  return true;
}

__global__ void __launch_bounds__(NUM_THREADS, 1) gemm_grouped_kernel(const __grid_constant__ GroupedParams gp) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~(uintptr_t)1023);
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + STAGES * STAGE_BYTES);
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 2 * STAGES + 4);
  __shared__ int s_abort[2];     // {abort, extra wait in ms}: see bw::mbar_wait

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const uint32_t smem_base = bw::smem_u32(smem);
  const uint32_t bar_base = bw::smem_u32(bars);
  auto full_bar = [&](int s) { return bar_base + 8u * s; };
  auto empty_bar = [&](int s) { return bar_base + 8u * (STAGES + s); };
  auto tfull_bar = [&](int a) { return bar_base + 8u * (2 * STAGES + a); };
  auto tempty_bar = [&](int a) { return bar_base + 8u * (2 * STAGES + 2 + a); };
  const int item_begin = gp.offsets[blockIdx.x], item_end = gp.offsets[blockIdx.x + 1];

  if (threadIdx.x == 0) {
    s_abort[0] = 0;
    s_abort[1] = 0;
    for (int s = 0; s < STAGES; s++) {
      bw::mbar_init(full_bar(s), 1);
      bw::mbar_init(empty_bar(s), 1);
    }
    for (int a = 0; a < 2; a++) {
      bw::mbar_init(tfull_bar(a), 1);
      bw::mbar_init(tempty_bar(a), 4);
    }
    bw::mbar_init_fence();
  }
  if (warp == 1) bw::tmem_alloc(bw::smem_u32(tmem_slot), 512);
  bw::fence_before();
  __syncthreads();
  bw::fence_after();
  const uint32_t tmem_base = *tmem_slot;
  volatile int* abort_flag = s_abort;

  if (warp == 0) {
    // ------------------------------ TMA producer ------------------------------
    if (lane == 0) {
      int stage = 0;
      uint32_t phase = 0;
      bool ok = true;
      int next_item = item_begin < item_end ? gp.items[item_begin] : 0;
      for (int it = item_begin; it < item_end && ok; it++) {
        const int item = next_item;
        if (it + 1 < item_end) next_item = gp.items[it + 1];      // in flight while this tile streams
        const int pi = item >> 24;
        const CUtensorMap* ta = &gp.ta[pi];
        const CUtensorMap* tb = &gp.tb[pi];
        int tm, tn;
        tile_coords(item & 0xFFFFFF, gp.prob[pi], tm, tn);
        const int split = gp.prob[pi].epi == 1 ? gp.prob[pi].half : 0;
        const int m0 = tm * BM, n0 = split ? tn * (BN / 2) : tn * BN;
        const int num_kb = gp.prob[pi].num_kb;
        switch (gp.prob[pi].a_mn * 2 + gp.prob[pi].b_mn) {
          case 0: ok = produce_tile<false, false>(ta, tb, m0, n0, num_kb, smem_base, bar_base, stage, phase, abort_flag, 0, split); break;
          case 1: ok = produce_tile<false, true>(ta, tb, m0, n0, num_kb, smem_base, bar_base, stage, phase, abort_flag); break;
          case 2: ok = produce_tile<true, false>(ta, tb, m0, n0, num_kb, smem_base, bar_base, stage, phase, abort_flag, 0, split); break;
          default: ok = produce_tile<true, true>(ta, tb, m0, n0, num_kb, smem_base, bar_base, stage, phase, abort_flag); break;
        }
        if (!ok) give_up(abort_flag, 1u);
      }
    }
  } else if (warp == 1) {
    // ------------------------------ MMA issuer ------------------------------
    if (lane == 0) {
      int stage = 0;
      uint32_t phase = 0;
      bool ok = true;
      int n = 0;
      int next_item = item_begin < item_end ? gp.items[item_begin] : 0;
      for (int it = item_begin; it < item_end && ok; it++, n++) {
        const int pi = next_item >> 24;
        if (it + 1 < item_end) next_item = gp.items[it + 1];
        const int num_kb = gp.prob[pi].num_kb;
        const int majors = gp.prob[pi].a_mn * 2 + gp.prob[pi].b_mn;
        const int acc = n & 1;
        const uint32_t acc_phase = (uint32_t)(n >> 1) & 1u;
        if (!bw::mbar_wait(tempty_bar(acc), acc_phase ^ 1u, abort_flag)) { give_up(abort_flag, 2u); ok = false; break; }
        bw::fence_after();
        const uint32_t d_tmem = tmem_base + (uint32_t)acc * BN;
        switch (majors) {
          case 0: ok = mma_tile<false, false>(d_tmem, num_kb, smem_base, bar_base, stage, phase, abort_flag); break;
          case 1: ok = mma_tile<false, true>(d_tmem, num_kb, smem_base, bar_base, stage, phase, abort_flag); break;
          case 2: ok = mma_tile<true, false>(d_tmem, num_kb, smem_base, bar_base, stage, phase, abort_flag); break;
          default: ok = mma_tile<true, true>(d_tmem, num_kb, smem_base, bar_base, stage, phase, abort_flag); break;
        }
        if (ok) bw::umma_commit(tfull_bar(acc));          // accumulator complete
        else give_up(abort_flag, 3u);
      }
    }
  } else {
    // ------------------------------ epilogue (4 warps) ------------------------------
    const int quad = warp & 3;
    int n = 0;
    int next_item = item_begin < item_end ? gp.items[item_begin] : 0;
    for (int it = item_begin; it < item_end; it++, n++) {
      const int item = next_item;
      if (it + 1 < item_end) next_item = gp.items[it + 1];
      const int pi = item >> 24;
      int tm, tn;
      tile_coords(item & 0xFFFFFF, gp.prob[pi], tm, tn);
      const int pM = gp.prob[pi].M, pN = gp.prob[pi].N;
      const bool accumulate = gp.prob[pi].accumulate != 0;
      bf16* const pC = gp.prob[pi].C;
      const long long ldc = gp.prob[pi].ldc;
      const int acc = n & 1;
      const uint32_t acc_phase = (uint32_t)(n >> 1) & 1u;
      const int row = tm * BM + quad * 32 + lane;
      const int n0 = tn * BN;
      if (gp.prob[pi].epi == 2 && row < pM) {
        // while the MMAs of this tile run: pull the g | u values its epilogue will read into L2
        const bf16* pre = gp.prob[pi].C2 + (size_t)row * gp.prob[pi].ldc2 + n0;
        const int half = gp.prob[pi].half;
#pragma unroll
        for (int l = 0; l < BN / 64; l++) {
          if (n0 + l * 64 < half) {
            asm volatile("prefetch.global.L2 [%0];" ::"l"(pre + l * 64));
            asm volatile("prefetch.global.L2 [%0];" ::"l"(pre + half + l * 64));
          }
        }
      }
      if (!bw::mbar_wait(tfull_bar(acc), acc_phase, abort_flag)) { give_up(abort_flag, 4u); break; }
      bw::fence_after();
      const uint32_t taddr = tmem_base + ((uint32_t)(quad * 32) << 16) + (uint32_t)acc * BN;
      bf16* crow = pC + (size_t)row * ldc + n0;
      const int epi = gp.prob[pi].epi;
      if (epi == 1) {
        // gate | up tile: store both, and silu(g) * u computed from the ROUNDED values (what a
        // separate pass over the stored matrix would see, and what the backward recomputes from)
        const int half = gp.prob[pi].half;
        const int c0 = tn * (BN / 2);
        bf16* grow = pC + (size_t)row * ldc + c0;
        bf16* hrow = gp.prob[pi].C2 + (size_t)row * gp.prob[pi].ldc2 + c0;
#pragma unroll 1
        for (int c = 0; c < BN / 64; c++) {
          uint32_t rg[32], ru[32];
          bw::tmem_ld32(taddr + c * 32, rg);
          bw::tmem_ld32(taddr + BN / 2 + c * 32, ru);
          bw::tmem_ld_wait();
          if (row < pM) {
#pragma unroll
            for (int g = 0; g < 4; g++) {
              if (c0 + c * 32 + g * 8 < half) {
                float fg[8], fu[8], h[8];
#pragma unroll
                for (int i = 0; i < 8; i++) { fg[i] = __uint_as_float(rg[g * 8 + i]); fu[i] = __uint_as_float(ru[g * 8 + i]); }
                const uint4 pg = pack8(fg), pu = pack8(fu);
                *reinterpret_cast<uint4*>(grow + c * 32 + g * 8) = pg;
                *reinterpret_cast<uint4*>(grow + half + c * 32 + g * 8) = pu;
                unpack8(pg, fg);
                unpack8(pu, fu);
#pragma unroll
                for (int i = 0; i < 8; i++) h[i] = fg[i] / (1.f + __expf(-fg[i])) * fu[i];
                *reinterpret_cast<uint4*>(hrow + c * 32 + g * 8) = pack8(h);
              }
            }
          }
        }
        bw::fence_before();
        __syncwarp();
        if (lane == 0) bw::mbar_arrive(tempty_bar(acc));
        continue;
      }
      if (epi == 2) {
        // dh tile of the down projection -> dg | du, with g | u read from C2.  The 8 loads of a
        // 32-column chunk are issued together, and the chunk after it is already in flight, before
        // anything is stored (a store in between would order the loads behind it).
        const int half = gp.prob[pi].half;
        const bf16* gurow = gp.prob[pi].C2 + (size_t)row * gp.prob[pi].ldc2 + n0;
        const bool row_ok = row < pM;
        uint4 gq[2][4], uq[2][4];
        auto fetch = [&](int c, int buf) {
#pragma unroll
          for (int g = 0; g < 4; g++) {
            const bool ok = row_ok && (n0 + c * 32 + g * 8 < half);
            gq[buf][g] = ok ? __ldg(reinterpret_cast<const uint4*>(gurow + c * 32 + g * 8)) : make_uint4(0, 0, 0, 0);
            uq[buf][g] = ok ? __ldg(reinterpret_cast<const uint4*>(gurow + half + c * 32 + g * 8)) : make_uint4(0, 0, 0, 0);
          }
        };
        fetch(0, 0);
#pragma unroll
        for (int c = 0; c < BN / 32; c++) {
          if (c + 1 < BN / 32) fetch(c + 1, (c + 1) & 1);
          uint32_t r[32];
          bw::tmem_ld32(taddr + c * 32, r);
          bw::tmem_ld_wait();
          if (row_ok) {
#pragma unroll
            for (int g = 0; g < 4; g++) {
              if (n0 + c * 32 + g * 8 < half) {
                float d[8], fg[8], fu[8], dg[8], du[8];
#pragma unroll
                for (int i = 0; i < 8; i++) d[i] = __uint_as_float(r[g * 8 + i]);
                unpack8(pack8(d), d);                 // the value a stored bf16 dh would have had
                unpack8(gq[c & 1][g], fg);
                unpack8(uq[c & 1][g], fu);
#pragma unroll
                for (int i = 0; i < 8; i++) {
                  const float sig = 1.f / (1.f + __expf(-fg[i]));
                  dg[i] = d[i] * fu[i] * sig * (1.f + fg[i] * (1.f - sig));
                  du[i] = d[i] * fg[i] * sig;
                }
                *reinterpret_cast<uint4*>(crow + c * 32 + g * 8) = pack8(dg);
                *reinterpret_cast<uint4*>(crow + half + c * 32 + g * 8) = pack8(du);
              }
            }
          }
        }
        bw::fence_before();
        __syncwarp();
        if (lane == 0) bw::mbar_arrive(tempty_bar(acc));
        continue;
      }
#pragma unroll 1
      for (int c = 0; c < BN / 32; c++) {
        uint32_t r[32];
        bw::tmem_ld32(taddr + c * 32, r);
        bw::tmem_ld_wait();
        if (row < pM) {
#pragma unroll
          for (int g = 0; g < 4; g++) {
            const int col = n0 + c * 32 + g * 8;
            if (col < pN) {
              float f[8];
#pragma unroll
              for (int i = 0; i < 8; i++) f[i] = __uint_as_float(r[g * 8 + i]);
              uint4* dst = reinterpret_cast<uint4*>(crow + c * 32 + g * 8);
              if (accumulate) {
                float o[8];
                unpack8(*dst, o);
#pragma unroll
                for (int i = 0; i < 8; i++) f[i] += o[i];
              }
              *dst = pack8(f);
            }
          }
        }
      }
      bw::fence_before();
      __syncwarp();
      if (lane == 0) bw::mbar_arrive(tempty_bar(acc));
    }
  }

  bw::fence_before();
  __syncthreads();
  if (warp == 1) {
    bw::fence_after();
    bw::tmem_dealloc(tmem_base, 512);
  }
}

// ---- ragged variant: row segments whose sizes live in device memory --------------------------------
// The per-expert GEMMs of a MoE layer.  One activation buffer [cap, K] holds the rows of all local
// experts, expert e in rows [seg[e], seg[e] + seg[LE + e]); every segment starts on a multiple of
// 128 rows and the rows between a segment's end and the next multiple of 128 are zero.  Offsets and
// counts are written by the planning kernel of the token exchange (moe.cu) and are never read on
// the host: every role of every CTA derives the same tile list from them.
//   mode 0   C[rows of e, N] = A[rows of e, K] . op(B_e)^T           (forward, data gradient)
//            all tiles cost the same, so CTA c simply takes tiles c, c + grid, ...
//   mode 1   C_e[Nw, Kw] (+)= A[rows of e, Nw]^T . B[rows of e, Kw]  (weight gradient; the reduction
//            runs over the rows of the segment, in 64-row steps, padding rows contribute zeros)
// Before its first load the producer can wait (bounded) for an arrival word: the rows are pushed
// into A by other GPUs.
struct RaggedParams {
  CUtensorMap ta;                      // mode 0: [cap, K] K-major;  mode 1: [cap, Nw] as MN-major A
  CUtensorMap tb[MAX_PROBLEMS];        // mode 0: B_e;               mode 1: tb[0] = [cap, Kw] as MN-major B
  bf16* C[MAX_PROBLEMS];               // mode 0: C[0] = common [cap, N];  mode 1: C_e
  long long ldc;
  const int* seg;
  int LE, M_w, N, K, b_mn, mode, accumulate, cap;
  int tiles_n, tiles_m_w, num_kb;
  const unsigned int* wait_flag;
  unsigned int wait_target;
  unsigned long long wait_ns;
};

struct RaggedTile { int e, m0, n0, num_kb, k_base; };

// Tile `t` of the launch, or e < 0 past the end.  seg_* are the CTA's shared copies of the table.
__device__ __forceinline__ RaggedTile ragged_tile(int t, const RaggedParams& rp, const int* s_off, const int* s_tiles) {
  RaggedTile r;
  r.e = -1; r.m0 = r.n0 = r.num_kb = r.k_base = 0;
  if (rp.mode == 0) {
    for (int e = 0; e < rp.LE; e++) {
      const int nt = s_tiles[e] * rp.tiles_n;
      if (t < nt) {
        Problem pr;
        pr.tiles_m = s_tiles[e]; pr.tiles_n = rp.tiles_n;
        int tm, tn;
        tile_coords(t, pr, tm, tn);
        r.e = e; r.m0 = s_off[e] + tm * BM; r.n0 = tn * BN; r.num_kb = rp.num_kb;
        return r;
      }
      t -= nt;
    }
  } else {
    const int per = rp.tiles_m_w * rp.tiles_n;
    const int e = t / per;
    if (e < rp.LE) {
      const int tt = t - e * per;
      r.e = e; r.m0 = (tt % rp.tiles_m_w) * BM; r.n0 = (tt / rp.tiles_m_w) * BN;
      r.num_kb = s_tiles[e];              // 64-row steps over the segment
      r.k_base = s_off[e];
    }
  }
  return r;
}

__global__ void __launch_bounds__(NUM_THREADS, 1) gemm_ragged_kernel(const __grid_constant__ RaggedParams rp) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~(uintptr_t)1023);
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + STAGES * STAGE_BYTES);
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 2 * STAGES + 4);
  __shared__ int s_abort[2];     // {abort, extra wait in ms}: see bw::mbar_wait
  __shared__ int s_off[MAX_PROBLEMS], s_tiles[MAX_PROBLEMS];

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const uint32_t smem_base = bw::smem_u32(smem);
  const uint32_t bar_base = bw::smem_u32(bars);
  auto full_bar = [&](int s) { return bar_base + 8u * s; };
  auto empty_bar = [&](int s) { return bar_base + 8u * (STAGES + s); };
  auto tfull_bar = [&](int a) { return bar_base + 8u * (2 * STAGES + a); };
  auto tempty_bar = [&](int a) { return bar_base + 8u * (2 * STAGES + 2 + a); };

  if (threadIdx.x == 0) {
    s_abort[0] = 0;
    s_abort[1] = rp.wait_flag ? bw::wait_extra_ms(rp.wait_ns) : 0;
    for (int s = 0; s < STAGES; s++) {
      bw::mbar_init(full_bar(s), 1);
      bw::mbar_init(empty_bar(s), 1);
    }
    for (int a = 0; a < 2; a++) {
      bw::mbar_init(tfull_bar(a), 1);
      bw::mbar_init(tempty_bar(a), 4);
    }
    bw::mbar_init_fence();
  }
  if (threadIdx.x < rp.LE) {
    // segment table -> offsets and tile (mode 0: 128-row tiles) / step (mode 1: 64-row steps) counts,
    // clamped so that no coordinate can pass the end of the buffer
    int off = rp.seg[threadIdx.x], cnt = rp.seg[rp.LE + threadIdx.x];
    if (off < 0 || off > rp.cap) { off = 0; cnt = 0; }
    if (cnt < 0) cnt = 0;
    if (off + cnt > rp.cap) cnt = rp.cap - off;
    s_off[threadIdx.x] = off;
    s_tiles[threadIdx.x] = rp.mode == 0 ? (cnt + BM - 1) / BM : (cnt + BK - 1) / BK;
  }
  if (warp == 1) bw::tmem_alloc(bw::smem_u32(tmem_slot), 512);
  bw::fence_before();
  __syncthreads();
  bw::fence_after();
  const uint32_t tmem_base = *tmem_slot;
  volatile int* abort_flag = s_abort;

  if (warp == 0) {
    // ------------------------------ TMA producer ------------------------------
    if (lane == 0) {
      int stage = 0;
      uint32_t phase = 0;
      bool ok = true;
      if (rp.wait_flag) {
        // the rows of A are pushed by other GPUs: acquire the arrival word, then order their
        // generic-proxy writes before the TMA (async proxy) reads
        if (!lbcomm::flag_wait_ge(rp.wait_flag, rp.wait_target, rp.wait_ns)) { give_up(abort_flag, 11u); ok = false; }
        asm volatile("fence.proxy.async;" ::: "memory");
      }
      for (int t = blockIdx.x; ok; t += gridDim.x) {
        const RaggedTile rt = ragged_tile(t, rp, s_off, s_tiles);
        if (rt.e < 0) break;
        if (rt.num_kb == 0) continue;
        if (rp.mode == 0) {
          if (!rp.b_mn) ok = produce_tile<false, false>(&rp.ta, &rp.tb[rt.e], rt.m0, rt.n0, rt.num_kb, smem_base, bar_base, stage, phase, abort_flag);
          else          ok = produce_tile<false, true>(&rp.ta, &rp.tb[rt.e], rt.m0, rt.n0, rt.num_kb, smem_base, bar_base, stage, phase, abort_flag);
        } else {
          ok = produce_tile<true, true>(&rp.ta, &rp.tb[0], rt.m0, rt.n0, rt.num_kb, smem_base, bar_base, stage, phase, abort_flag, rt.k_base);
        }
        if (!ok) give_up(abort_flag, 1u);
      }
    }
  } else if (warp == 1) {
    // ------------------------------ MMA issuer ------------------------------
    if (lane == 0) {
      int stage = 0;
      uint32_t phase = 0;
      bool ok = true;
      int n = 0;
      for (int t = blockIdx.x; ok; t += gridDim.x) {
        const RaggedTile rt = ragged_tile(t, rp, s_off, s_tiles);
        if (rt.e < 0) break;
        if (rt.num_kb == 0) continue;
        const int acc = n & 1;
        const uint32_t acc_phase = (uint32_t)(n >> 1) & 1u;
        if (!bw::mbar_wait(tempty_bar(acc), acc_phase ^ 1u, abort_flag)) { give_up(abort_flag, 2u); ok = false; break; }
        bw::fence_after();
        const uint32_t d_tmem = tmem_base + (uint32_t)acc * BN;
        if (rp.mode == 0) {
          if (!rp.b_mn) ok = mma_tile<false, false>(d_tmem, rt.num_kb, smem_base, bar_base, stage, phase, abort_flag);
          else          ok = mma_tile<false, true>(d_tmem, rt.num_kb, smem_base, bar_base, stage, phase, abort_flag);
        } else {
          ok = mma_tile<true, true>(d_tmem, rt.num_kb, smem_base, bar_base, stage, phase, abort_flag);
        }
        if (ok) bw::umma_commit(tfull_bar(acc));
        else give_up(abort_flag, 3u);
        n++;
      }
    }
  } else {
    // ------------------------------ epilogue (4 warps) ------------------------------
    const int quad = warp & 3;
    int n = 0;
    for (int t = blockIdx.x;; t += gridDim.x) {
      const RaggedTile rt = ragged_tile(t, rp, s_off, s_tiles);
      if (rt.e < 0) break;
      if (rt.num_kb == 0) continue;
      const int acc = n & 1;
      const uint32_t acc_phase = (uint32_t)(n >> 1) & 1u;
      if (!bw::mbar_wait(tfull_bar(acc), acc_phase, abort_flag)) { give_up(abort_flag, 4u); break; }
      bw::fence_after();
      const int row = rt.m0 + quad * 32 + lane;
      const int row_end = rp.mode == 0 ? rp.cap : rp.M_w;      // mode 0 writes whole 128-row tiles (padding rows are zeros)
      bf16* const pC = rp.mode == 0 ? rp.C[0] : rp.C[rt.e];
      const bool accumulate = rp.accumulate != 0;
      const uint32_t taddr = tmem_base + ((uint32_t)(quad * 32) << 16) + (uint32_t)acc * BN;
      bf16* crow = pC + (size_t)row * rp.ldc + rt.n0;
#pragma unroll 1
      for (int c = 0; c < BN / 32; c++) {
        uint32_t r[32];
        bw::tmem_ld32(taddr + c * 32, r);
        bw::tmem_ld_wait();
        if (row < row_end) {
#pragma unroll
          for (int g = 0; g < 4; g++) {
            const int col = rt.n0 + c * 32 + g * 8;
            if (col < rp.N) {
              float f[8];
#pragma unroll
              for (int i = 0; i < 8; i++) f[i] = __uint_as_float(r[g * 8 + i]);
              uint4* dst = reinterpret_cast<uint4*>(crow + c * 32 + g * 8);
              if (accumulate) {
                float o[8];
                unpack8(*dst, o);
#pragma unroll
                for (int i = 0; i < 8; i++) f[i] += o[i];
              }
              *dst = pack8(f);
            }
          }
        }
      }
      bw::fence_before();
      __syncwarp();
      if (lane == 0) bw::mbar_arrive(tempty_bar(acc));
      n++;
    }
  }

  bw::fence_before();
  __syncthreads();
  if (warp == 1) {
    bw::fence_after();
    bw::tmem_dealloc(tmem_base, 512);
  }
}

// ---- host side: static schedule, cached per (device, shapes) -------------------------------------
struct Schedule {
  int grid = 0;
  int* d_offsets = nullptr;
  int* d_items = nullptr;
  unsigned long long last_use = 0;
};
// Cache of uploaded schedules, keyed by (device, M, N, K of every problem).  A training run uses a
// few dozen shape sets; callers whose row counts change from call to call (expert-parallel MoE)
// use lb_gemm_ragged instead, which takes the counts from device memory and needs no schedule.
// The cache is still bounded: beyond MAX_SCHEDULES entries the least recently used one is freed.
constexpr size_t MAX_SCHEDULES = 128;
std::map<std::vector<int>, Schedule> g_schedules;
unsigned long long g_sched_clock = 0;
std::mutex g_sched_mutex;
int g_sms = 0;

// Longest tiles first, each to the least loaded CTA (ties: lowest CTA index, which keeps tiles
// that run at the same time adjacent in the problem's L2-friendly order).
struct Item { int cost, code; };

// The assignment itself (host only): per-CTA item lists, longest tiles first, each to the least
// loaded CTA.  Returns the load (in k-block units) of the busiest CTA.
long long assign_items(const Problem* probs, int np, int sms, std::vector<std::vector<int>>* per_out, int* total_out,
                       long long* work_out) {
  std::vector<Item> items;
  std::vector<int> order(np);
  for (int i = 0; i < np; i++) order[i] = i;
  std::stable_sort(order.begin(), order.end(), [&](int a, int b) { return probs[a].num_kb > probs[b].num_kb; });
  long long work = 0;
  for (int oi = 0; oi < np; oi++) {
    const int i = order[oi];
    const int nt = probs[i].tiles_m * probs[i].tiles_n;
    if (nt >= (1 << 24)) return -1;
    for (int t = 0; t < nt; t++) {
      items.push_back({probs[i].num_kb + 6, (i << 24) | t});   // +6: fixed cost per tile
      work += probs[i].num_kb + 6;
    }
  }
  const int total = (int)items.size();
  const int grid = total < sms ? total : sms;
  typedef std::pair<long long, int> Load;
  std::priority_queue<Load, std::vector<Load>, std::greater<Load>> heap;
  for (int c = 0; c < grid; c++) heap.push({0, c});
  std::vector<std::vector<int>> per(grid);
  long long busiest = 0;
  for (const Item& it : items) {
    Load l = heap.top();
    heap.pop();
    per[l.second].push_back(it.code);
    const long long load = l.first + it.cost;
    if (load > busiest) busiest = load;
    heap.push({load, l.second});
  }
  if (per_out) per_out->swap(per);
  if (total_out) *total_out = total;
  if (work_out) *work_out = work;
  return busiest;
}

int build_schedule(const Problem* probs, int np, int sms, Schedule* out) {
  std::vector<std::vector<int>> per;
  int total = 0;
  if (assign_items(probs, np, sms, &per, &total, nullptr) < 0) return LB_ERR_SHAPE;
  const int grid = (int)per.size();
  std::vector<int> offsets(grid + 1, 0), flat;
  flat.reserve(total);
  for (int c = 0; c < grid; c++) {
    offsets[c] = (int)flat.size();
    flat.insert(flat.end(), per[c].begin(), per[c].end());
  }
  offsets[grid] = (int)flat.size();
  if (cudaMalloc(&out->d_offsets, sizeof(int) * (grid + 1)) != cudaSuccess) return LB_ERR_LAUNCH;
  if (cudaMalloc(&out->d_items, sizeof(int) * (total > 0 ? total : 1)) != cudaSuccess) return LB_ERR_LAUNCH;
  cudaMemcpy(out->d_offsets, offsets.data(), sizeof(int) * (grid + 1), cudaMemcpyHostToDevice);
  cudaMemcpy(out->d_items, flat.data(), sizeof(int) * total, cudaMemcpyHostToDevice);
  out->grid = grid;
  return LB_OK;
}

}  // namespace

// Copies the status words of the grouped GEMM kernel to host memory and clears them.
extern "C" int lb_gemm_grouped_status(void* out) {
  cudaError_t e = cudaMemcpyFromSymbol(out, g_grp_status, sizeof(unsigned int) * 4);
  if (e != cudaSuccess) { g_lb_last_cuda_error = (int)e; return LB_ERR_LAUNCH; }
  unsigned int zeros[4] = {0, 0, 0, 0};
  cudaMemcpyToSymbol(g_grp_status, zeros, sizeof(zeros));
  return LB_OK;
}

// Host only (no CUDA call): the schedule lb_gemm_grouped would build for these shapes on `sms` SMs.
// out[0] = load of the busiest CTA, out[1] = total work, out[2] = number of CTAs used, all in k-block
// units of 64 (a tile counts its k-blocks + 6).  busiest * CTAs / total is the imbalance factor.
// Number of schedules currently cached (never more than MAX_SCHEDULES).
extern "C" int lb_gemm_grouped_cached() {
  std::lock_guard<std::mutex> lock(g_sched_mutex);
  return (int)g_schedules.size();
}

extern "C" int lb_gemm_grouped_plan(int n, const int* M, const int* N, const int* K, int sms, long long* out) {
  if (n < 1 || n > MAX_PROBLEMS || sms < 1) return LB_ERR_SHAPE;
  Problem probs[MAX_PROBLEMS];
  for (int i = 0; i < n; i++) {
    if (M[i] <= 0 || N[i] <= 0 || K[i] <= 0) return LB_ERR_SHAPE;
    probs[i].tiles_m = (M[i] + BM - 1) / BM; probs[i].tiles_n = (N[i] + BN - 1) / BN; probs[i].num_kb = (K[i] + BK - 1) / BK;
  }
  std::vector<std::vector<int>> per;
  int total = 0;
  long long work = 0;
  const long long busiest = assign_items(probs, n, sms, &per, &total, &work);
  if (busiest < 0) return LB_ERR_SHAPE;
  out[0] = busiest; out[1] = work; out[2] = (long long)per.size();
  return LB_OK;
}

// n problems (1..8), arrays of length n.  Per problem the rules of lb_gemm_bf16 apply: pointers
// 16-byte aligned, lda / ldb / ldc / N multiples of 8 (M too when a_mn).  accumulate[i] != 0 adds
// the product to the old contents of C_i.  The first call with a new set of shapes builds and
// uploads the schedule (two small device allocations, synchronous copies); later calls only launch.
//
// lb_gemm_grouped_epi additionally takes, per problem, an epilogue selector (see `Problem`), a second
// matrix C2 with its leading dimension, and `half`:
//   epi 1: B is a fused [2 * half, K] gate | up weight (b_mn = 0), N = 2 * half, C [M, 2 * half] receives
//          g | u and C2 [M, half] receives silu(g) * u;
//   epi 2: N = half, the product is dh; C2 [M, 2 * half] holds g | u and C [M, 2 * half] receives dg | du.
extern "C" int lb_gemm_grouped_epi(int n, const void* const* A, const void* const* B, void* const* C, const int* M,
                                   const int* N, const int* K, const long long* lda, const long long* ldb,
                                   const long long* ldc, const int* a_mn, const int* b_mn, const int* accumulate,
                                   const int* epi, void* const* C2, const long long* ldc2, const int* half,
                                   void* stream) {
  if (n < 1 || n > MAX_PROBLEMS) return LB_ERR_SHAPE;
  static thread_local GroupedParams gp;         // 2.5 KB of tensor maps: kept off the stack, one per calling thread
  std::vector<int> key;
  int dev = 0;
  cudaGetDevice(&dev);
  key.push_back(dev);
  for (int i = 0; i < n; i++) {
    if (M[i] <= 0 || N[i] <= 0 || K[i] <= 0) return LB_ERR_SHAPE;
    if ((lda[i] % 8) || (ldb[i] % 8) || (ldc[i] % 8) || (N[i] % 8) || (a_mn[i] && (M[i] % 8))) return LB_ERR_SHAPE;
    if (((uintptr_t)A[i] | (uintptr_t)B[i] | (uintptr_t)C[i]) & 15) return LB_ERR_ARG;
    int rc;
    if (!a_mn[i]) rc = bw::make_map_bf16(&gp.ta[i], A[i], (uint64_t)K[i], (uint64_t)M[i], (uint64_t)lda[i], BK, BM);
    else          rc = bw::make_map_bf16(&gp.ta[i], A[i], (uint64_t)M[i], (uint64_t)K[i], (uint64_t)lda[i], 64, BK);
    if (rc) return rc;
    const int e = epi ? epi[i] : 0;
    if (e < 0 || e > 2) return LB_ERR_ARG;
    if (e) {
      if (!C2 || !ldc2 || !half || !C2[i] || ((uintptr_t)C2[i] & 15) || (ldc2[i] % 8) || half[i] <= 0 || (half[i] % 8)) return LB_ERR_ARG;
      if (e == 1 && (b_mn[i] || N[i] != 2 * half[i])) return LB_ERR_SHAPE;
      if (e == 2 && N[i] != half[i]) return LB_ERR_SHAPE;
      if (accumulate && accumulate[i]) return LB_ERR_ARG;
    }
    if (!b_mn[i]) rc = bw::make_map_bf16(&gp.tb[i], B[i], (uint64_t)K[i], (uint64_t)N[i], (uint64_t)ldb[i], BK, e == 1 ? BN / 2 : BN);
    else          rc = bw::make_map_bf16(&gp.tb[i], B[i], (uint64_t)N[i], (uint64_t)K[i], (uint64_t)ldb[i], 64, BK);
    if (rc) return rc;
    Problem& p = gp.prob[i];
    p.C = (bf16*)C[i]; p.ldc = ldc[i]; p.M = M[i]; p.N = N[i]; p.K = K[i];
    p.C2 = e ? (bf16*)C2[i] : nullptr; p.ldc2 = e ? ldc2[i] : 0; p.epi = e; p.half = e ? half[i] : 0;
    p.a_mn = a_mn[i]; p.b_mn = b_mn[i]; p.accumulate = accumulate ? accumulate[i] : 0;
    p.tiles_m = (M[i] + BM - 1) / BM; p.tiles_n = (N[i] + BN - 1) / BN; p.num_kb = (K[i] + BK - 1) / BK;
    key.push_back(M[i]); key.push_back(N[i]); key.push_back(K[i]);
  }
  {
    std::lock_guard<std::mutex> lock(g_sched_mutex);
    if (g_sms == 0) {
      cudaDeviceGetAttribute(&g_sms, cudaDevAttrMultiProcessorCount, dev);
      cudaFuncSetAttribute(gemm_grouped_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, SMEM_BYTES);
    }
  }
  Schedule sched;
  {
    std::lock_guard<std::mutex> lock(g_sched_mutex);
    auto it = g_schedules.find(key);
    if (it == g_schedules.end()) {
      if (g_schedules.size() >= MAX_SCHEDULES) {
        // evict the least recently used entry; cudaFree waits for kernels that may still read it
        auto victim = g_schedules.begin();
        for (auto j = g_schedules.begin(); j != g_schedules.end(); ++j)
          if (j->second.last_use < victim->second.last_use) victim = j;
        cudaFree(victim->second.d_offsets);
        cudaFree(victim->second.d_items);
        g_schedules.erase(victim);
      }
      Schedule s;
      int rc = build_schedule(gp.prob, n, g_sms, &s);
      if (rc) return rc;
      it = g_schedules.emplace(key, s).first;
    }
    it->second.last_use = ++g_sched_clock;
    sched = it->second;
  }
  gp.offsets = sched.d_offsets;
  gp.items = sched.d_items;
  gemm_grouped_kernel<<<sched.grid, NUM_THREADS, SMEM_BYTES, (cudaStream_t)stream>>>(gp);
  LB_CHECK_LAUNCH();
  return LB_OK;
}


extern "C" int lb_gemm_grouped(int n, const void* const* A, const void* const* B, void* const* C, const int* M,
                               const int* N, const int* K, const long long* lda, const long long* ldb,
                               const long long* ldc, const int* a_mn, const int* b_mn, const int* accumulate,
                               void* stream) {
  return lb_gemm_grouped_epi(n, A, B, C, M, N, K, lda, ldb, ldc, a_mn, b_mn, accumulate, nullptr, nullptr, nullptr, nullptr,
                             stream);
}

// Expert GEMMs over ragged row segments (see gemm_ragged_kernel).  seg: device table of 2 * LE + 2
// ints (offsets, counts, ...), LE <= 8 local experts.
//  mode 0: C [cap, N] = A [cap, K] . op(B_e)^T per segment; B: host array of LE weight pointers
//          ([N, K], or [K, N] with b_mn), all with leading dimension ldb.  wait_flag (or null): device
//          word that must reach wait_target before A is read.
extern "C" int lb_gemm_ragged(const void* A, const void* const* B, void* C, const void* seg, int LE, int cap, int N, int K,
                              long long lda, long long ldb, long long ldc, int b_mn, const void* wait_flag,
                              unsigned int wait_target, void* stream) {
  if (LE < 1 || LE > MAX_PROBLEMS || cap <= 0 || N <= 0 || K <= 0) return LB_ERR_SHAPE;
  if ((lda % 8) || (ldb % 8) || (ldc % 8) || (N % 8) || (K % 8)) return LB_ERR_SHAPE;
  if (((uintptr_t)A | (uintptr_t)C) & 15) return LB_ERR_ARG;
  static thread_local RaggedParams rp;
  int rc = bw::make_map_bf16(&rp.ta, A, (uint64_t)K, (uint64_t)cap, (uint64_t)lda, BK, BM);
  if (rc) return rc;
  for (int e = 0; e < LE; e++) {
    if ((uintptr_t)B[e] & 15) return LB_ERR_ARG;
    if (!b_mn) rc = bw::make_map_bf16(&rp.tb[e], B[e], (uint64_t)K, (uint64_t)N, (uint64_t)ldb, BK, BN);
    else       rc = bw::make_map_bf16(&rp.tb[e], B[e], (uint64_t)N, (uint64_t)K, (uint64_t)ldb, 64, BK);
    if (rc) return rc;
    rp.C[e] = nullptr;
  }
  rp.C[0] = (bf16*)C; rp.ldc = ldc; rp.seg = (const int*)seg; rp.LE = LE; rp.M_w = 0; rp.N = N; rp.K = K; rp.b_mn = b_mn;
  rp.mode = 0; rp.accumulate = 0; rp.cap = cap;
  rp.tiles_n = (N + BN - 1) / BN; rp.tiles_m_w = 0; rp.num_kb = (K + BK - 1) / BK;
  rp.wait_flag = (const unsigned int*)wait_flag; rp.wait_target = wait_target; rp.wait_ns = g_lb_flag_wait_ns;
  {
    std::lock_guard<std::mutex> lock(g_sched_mutex);
    static bool attr = false;
    if (!attr) { cudaFuncSetAttribute(gemm_ragged_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, SMEM_BYTES); attr = true; }
  }
  gemm_ragged_kernel<<<lb_num_sms(), NUM_THREADS, SMEM_BYTES, (cudaStream_t)stream>>>(rp);
  LB_CHECK_LAUNCH();
  return LB_OK;
}

//  Weight gradients: C_e [Nw, Kw] (+)= dY[rows of e, Nw]^T . X[rows of e, Kw]; C: host array of LE
//  gradient pointers with leading dimension ldc.
extern "C" int lb_gemm_ragged_wgrad(const void* dY, const void* X, void* const* C, const void* seg, int LE, int cap, int Nw,
                                    int Kw, long long lddy, long long ldx, long long ldc, int accumulate, void* stream) {
  if (LE < 1 || LE > MAX_PROBLEMS || cap <= 0 || Nw <= 0 || Kw <= 0) return LB_ERR_SHAPE;
  if ((lddy % 8) || (ldx % 8) || (ldc % 8) || (Nw % 8) || (Kw % 8)) return LB_ERR_SHAPE;
  if (((uintptr_t)dY | (uintptr_t)X) & 15) return LB_ERR_ARG;
  static thread_local RaggedParams rp;
  int rc = bw::make_map_bf16(&rp.ta, dY, (uint64_t)Nw, (uint64_t)cap, (uint64_t)lddy, 64, BK);
  if (rc) return rc;
  rc = bw::make_map_bf16(&rp.tb[0], X, (uint64_t)Kw, (uint64_t)cap, (uint64_t)ldx, 64, BK);
  if (rc) return rc;
  for (int e = 0; e < LE; e++) {
    if ((uintptr_t)C[e] & 15) return LB_ERR_ARG;
    rp.C[e] = (bf16*)C[e];
  }
  rp.ldc = ldc; rp.seg = (const int*)seg; rp.LE = LE; rp.M_w = Nw; rp.N = Kw; rp.K = 0; rp.b_mn = 1; rp.mode = 1;
  rp.accumulate = accumulate; rp.cap = cap;
  rp.tiles_n = (Kw + BN - 1) / BN; rp.tiles_m_w = (Nw + BM - 1) / BM; rp.num_kb = 0;
  rp.wait_flag = nullptr; rp.wait_target = 0; rp.wait_ns = g_lb_flag_wait_ns;
  {
    std::lock_guard<std::mutex> lock(g_sched_mutex);
    static bool attr = false;
    if (!attr) { cudaFuncSetAttribute(gemm_ragged_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, SMEM_BYTES); attr = true; }
  }
  gemm_ragged_kernel<<<lb_num_sms(), NUM_THREADS, SMEM_BYTES, (cudaStream_t)stream>>>(rp);
  LB_CHECK_LAUNCH();
  return LB_OK;
}
