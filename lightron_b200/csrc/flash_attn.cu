// Causal / full softmax attention, forward and backward, FlashAttention-style (no S x S matrix in
// memory), bf16 in / fp32 accumulate, GQA by indexing (kv head = q head / (hq/hkv)).
//
// Layout: q [B, Sq, hq, d], k/v [B, Sk, hkv, d], o [B, Sq, hq, d]; the head dimension is
// contiguous, heads of a token are d apart, tokens are `*_ts` elements apart (so q, k, v may be
// column slices of one fused projection output) and batches are S * ts apart.
// lse [B, hq, Sq] holds log(sum exp(scale * s)) per row.
// causal: query i sees keys j <= i + (Sk - Sq) (bottom-right aligned, FlashAttention convention).
//
// This file is the warp-level mma.sync.m16n8k16 implementation (register accumulators,
// cp.async double buffering, ldmatrix fragments).
#include "common.cuh"

namespace {

__device__ __forceinline__ uint32_t smem_u32(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }

__device__ __forceinline__ void cp_async16(uint32_t dst, const void* src, bool valid) {
  const int sz = valid ? 16 : 0;  // src-size 0 => 16 zero bytes
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"(dst), "l"(src), "r"(sz) : "memory");
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
template <int N>
__device__ __forceinline__ void cp_async_wait() { asm volatile("cp.async.wait_group %0;" ::"n"(N) : "memory"); }

__device__ __forceinline__ void ldsm_x4(uint32_t addr, uint32_t& r0, uint32_t& r1, uint32_t& r2, uint32_t& r3) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];"
               : "=r"(r0), "=r"(r1), "=r"(r2), "=r"(r3) : "r"(addr));
}
__device__ __forceinline__ void ldsm_x4_t(uint32_t addr, uint32_t& r0, uint32_t& r1, uint32_t& r2, uint32_t& r3) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];"
               : "=r"(r0), "=r"(r1), "=r"(r2), "=r"(r3) : "r"(addr));
}
__device__ __forceinline__ void mma16816(float* c, const uint32_t* a, uint32_t b0, uint32_t b1) {
  asm volatile(
      "mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
      : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
      : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}
__device__ __forceinline__ uint32_t pack_bf16(float lo, float hi) {
  bf162 v = __floats2bfloat162_rn(lo, hi);
  return *reinterpret_cast<uint32_t*>(&v);
}

// Loads ROWS x D bf16 (row stride ts elements in global, PAD-padded rows in smem); rows >= n_valid
// are zero-filled.  All NT threads take part.
template <int ROWS, int D, int LDS, int NT>
__device__ __forceinline__ void load_tile(bf16* s, const bf16* g, long long ts, int n_valid) {
  constexpr int VPR = D / 8;
  for (int i = threadIdx.x; i < ROWS * VPR; i += NT) {
    const int r = i / VPR, c = i % VPR;
    const bool ok = r < n_valid;
    cp_async16(smem_u32(s + r * LDS + c * 8), g + (ok ? (long long)r * ts + c * 8 : 0), ok);
  }
}

struct FwdParams {
  const bf16 *q, *k, *v;
  bf16* o;
  float* lse;
  int B, Sq, Sk, hq, hkv;
  long long q_ts, k_ts, v_ts, o_ts;
  float scale;
  int causal;
};

// --------------------------------------------------------------------------------------------
// Forward.  CTA = 8 warps x 16 query rows = 128 rows; key blocks of 64, double buffered.
// --------------------------------------------------------------------------------------------
template <int D>
__global__ void __launch_bounds__(256, 1) flash_fwd_kernel(const FwdParams p) {
  constexpr int BM = 128, BN = 64, NT = 256, LDS = D + 8;
  extern __shared__ __align__(16) uint8_t smem_raw[];
  bf16* sQ = reinterpret_cast<bf16*>(smem_raw);
  bf16* sK = sQ + BM * LDS;           // [2][BN][LDS]
  bf16* sV = sK + 2 * BN * LDS;       // [2][BN][LDS]

  const int mb = gridDim.x - 1 - blockIdx.x;  // heavy (late) causal blocks first
  const int h = blockIdx.y, b = blockIdx.z;
  const int hk = h / (p.hq / p.hkv);
  const int m0 = mb * BM;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int g = lane >> 2, t = lane & 3;
  const int off = p.Sk - p.Sq;

  const bf16* qg = p.q + ((long long)b * p.Sq + m0) * p.q_ts + (long long)h * D;
  const bf16* kg = p.k + (long long)b * p.Sk * p.k_ts + (long long)hk * D;
  const bf16* vg = p.v + (long long)b * p.Sk * p.v_ts + (long long)hk * D;

  int n_blocks = (p.Sk + BN - 1) / BN;
  if (p.causal) {
    const int last = m0 + BM - 1 + off;  // largest visible key index for this query block
    n_blocks = min(n_blocks, last / BN + 1);
    if (last < 0) n_blocks = 0;
  }

  load_tile<BM, D, LDS, NT>(sQ, qg, p.q_ts, p.Sq - m0);
  if (n_blocks > 0) {
    load_tile<BN, D, LDS, NT>(sK, kg, p.k_ts, p.Sk);
    load_tile<BN, D, LDS, NT>(sV, vg, p.v_ts, p.Sk);
  }
  cp_async_commit();

  float o_acc[D / 8][4];
#pragma unroll
  for (int i = 0; i < D / 8; i++) o_acc[i][0] = o_acc[i][1] = o_acc[i][2] = o_acc[i][3] = 0.f;
  float m_i[2] = {-INFINITY, -INFINITY}, l_i[2] = {0.f, 0.f};
  const float sl2 = p.scale * 1.4426950408889634f;
  uint32_t qf[D / 16][4];

  for (int jb = 0; jb < n_blocks; jb++) {
    const int buf = jb & 1;
    cp_async_wait<0>();
    __syncthreads();
    if (jb + 1 < n_blocks) {  // prefetch the next K/V block into the other buffer
      const int n1 = (jb + 1) * BN;
      load_tile<BN, D, LDS, NT>(sK + (buf ^ 1) * BN * LDS, kg + (long long)n1 * p.k_ts, p.k_ts, p.Sk - n1);
      load_tile<BN, D, LDS, NT>(sV + (buf ^ 1) * BN * LDS, vg + (long long)n1 * p.v_ts, p.v_ts, p.Sk - n1);
      cp_async_commit();
    }
    if (jb == 0) {
#pragma unroll
      for (int kk = 0; kk < D / 16; kk++) {
        const int r = warp * 16 + (lane & 7) + ((lane >> 3) & 1) * 8;
        const int c = kk * 16 + (lane >> 4) * 8;
        ldsm_x4(smem_u32(sQ + r * LDS + c), qf[kk][0], qf[kk][1], qf[kk][2], qf[kk][3]);
      }
    }
    const bf16* sKb = sK + buf * BN * LDS;
    const bf16* sVb = sV + buf * BN * LDS;
    float s[BN / 8][4];
#pragma unroll
    for (int i = 0; i < BN / 8; i++) s[i][0] = s[i][1] = s[i][2] = s[i][3] = 0.f;
#pragma unroll
    for (int kk = 0; kk < D / 16; kk++) {
#pragma unroll
      for (int nt = 0; nt < BN / 16; nt++) {
        uint32_t b0, b1, b2, b3;
        const int n = nt * 16 + (lane & 7) + (lane >> 4) * 8;
        const int c = kk * 16 + ((lane >> 3) & 1) * 8;
        ldsm_x4(smem_u32(sKb + n * LDS + c), b0, b1, b2, b3);
        mma16816(s[2 * nt], qf[kk], b0, b1);
        mma16816(s[2 * nt + 1], qf[kk], b2, b3);
      }
    }
    // mask
    const int n0 = jb * BN;
    const int row0 = m0 + warp * 16 + g;
    const bool need_mask = (n0 + BN > p.Sk) || (p.causal && (n0 + BN - 1 > m0 + warp * 16 + off));
    if (need_mask) {
#pragma unroll
      for (int i = 0; i < BN / 8; i++) {
#pragma unroll
        for (int e = 0; e < 4; e++) {
          const int col = n0 + i * 8 + 2 * t + (e & 1);
          const int row = row0 + (e >> 1) * 8;
          if (col >= p.Sk || (p.causal && col > row + off)) s[i][e] = -INFINITY;
        }
      }
    }
    // online softmax (base-2 domain)
    float mx[2] = {m_i[0], m_i[1]};
#pragma unroll
    for (int i = 0; i < BN / 8; i++) {
      mx[0] = fmaxf(mx[0], fmaxf(s[i][0], s[i][1]));
      mx[1] = fmaxf(mx[1], fmaxf(s[i][2], s[i][3]));
    }
#pragma unroll
    for (int r = 0; r < 2; r++) {
      mx[r] = fmaxf(mx[r], __shfl_xor_sync(0xffffffffu, mx[r], 1));
      mx[r] = fmaxf(mx[r], __shfl_xor_sync(0xffffffffu, mx[r], 2));
    }
    float corr[2], msc[2];
#pragma unroll
    for (int r = 0; r < 2; r++) {
      msc[r] = (mx[r] == -INFINITY) ? 0.f : mx[r] * sl2;
      corr[r] = (m_i[r] == -INFINITY) ? 0.f : exp2f(m_i[r] * sl2 - msc[r]);
      m_i[r] = mx[r];
      l_i[r] *= corr[r];
    }
    float rs[2] = {0.f, 0.f};
#pragma unroll
    for (int i = 0; i < BN / 8; i++) {
      s[i][0] = exp2f(s[i][0] * sl2 - msc[0]);
      s[i][1] = exp2f(s[i][1] * sl2 - msc[0]);
      s[i][2] = exp2f(s[i][2] * sl2 - msc[1]);
      s[i][3] = exp2f(s[i][3] * sl2 - msc[1]);
      rs[0] += s[i][0] + s[i][1];
      rs[1] += s[i][2] + s[i][3];
    }
    l_i[0] += rs[0];
    l_i[1] += rs[1];
#pragma unroll
    for (int i = 0; i < D / 8; i++) {
      o_acc[i][0] *= corr[0]; o_acc[i][1] *= corr[0];
      o_acc[i][2] *= corr[1]; o_acc[i][3] *= corr[1];
    }
    // O += P V
#pragma unroll
    for (int kb = 0; kb < BN / 16; kb++) {
      uint32_t a[4];
      a[0] = pack_bf16(s[2 * kb][0], s[2 * kb][1]);
      a[1] = pack_bf16(s[2 * kb][2], s[2 * kb][3]);
      a[2] = pack_bf16(s[2 * kb + 1][0], s[2 * kb + 1][1]);
      a[3] = pack_bf16(s[2 * kb + 1][2], s[2 * kb + 1][3]);
#pragma unroll
      for (int dt = 0; dt < D / 16; dt++) {
        uint32_t b0, b1, b2, b3;
        const int kr = kb * 16 + (lane & 7) + ((lane >> 3) & 1) * 8;
        const int c = dt * 16 + (lane >> 4) * 8;
        ldsm_x4_t(smem_u32(sVb + kr * LDS + c), b0, b1, b2, b3);
        mma16816(o_acc[2 * dt], a, b0, b1);
        mma16816(o_acc[2 * dt + 1], a, b2, b3);
      }
    }
  }
  cp_async_wait<0>();
  __syncthreads();

  // finalize: quad-reduce the row sums, normalise, stage through smem (sQ region), 16-byte stores
#pragma unroll
  for (int r = 0; r < 2; r++) {
    l_i[r] += __shfl_xor_sync(0xffffffffu, l_i[r], 1);
    l_i[r] += __shfl_xor_sync(0xffffffffu, l_i[r], 2);
  }
  const float inv0 = l_i[0] > 0.f ? 1.f / l_i[0] : 0.f;
  const float inv1 = l_i[1] > 0.f ? 1.f / l_i[1] : 0.f;
  bf16* sO = sQ;
#pragma unroll
  for (int i = 0; i < D / 8; i++) {
    const int c = i * 8 + 2 * t;
    *reinterpret_cast<uint32_t*>(sO + (warp * 16 + g) * LDS + c) = pack_bf16(o_acc[i][0] * inv0, o_acc[i][1] * inv0);
    *reinterpret_cast<uint32_t*>(sO + (warp * 16 + g + 8) * LDS + c) = pack_bf16(o_acc[i][2] * inv1, o_acc[i][3] * inv1);
  }
  if (t == 0) {
#pragma unroll
    for (int r = 0; r < 2; r++) {
      const int row = m0 + warp * 16 + g + r * 8;
      if (row < p.Sq) {
        const float l = l_i[r];
        p.lse[((long long)b * p.hq + h) * p.Sq + row] = (l > 0.f) ? m_i[r] * p.scale + logf(l) : -INFINITY;
      }
    }
  }
  __syncthreads();
  bf16* og = p.o + ((long long)b * p.Sq + m0) * p.o_ts + (long long)h * D;
  constexpr int VPR = D / 8;
  for (int i = threadIdx.x; i < BM * VPR; i += NT) {
    const int r = i / VPR, c = i % VPR;
    if (m0 + r < p.Sq)
      *reinterpret_cast<uint4*>(og + (long long)r * p.o_ts + c * 8) = *reinterpret_cast<const uint4*>(sO + r * LDS + c * 8);
  }
}

// --------------------------------------------------------------------------------------------
// Backward.
//   delta[b,h,i] = sum_d o * do                                   (pre-pass)
//   CTA = (64-key block, kv head, batch), 4 warps x 16 key rows.  For every query head of the
//   group and every 64-query block that can see the key block:
//     S^T = K Q^T,  P^T = exp(scale S^T - lse),  dV += P^T dO,  dP^T = V dO^T,
//     dS^T = P^T (dP^T - delta) scale,  dK += dS^T Q,  dQ += dS K  (fp32 atomics into dq_acc)
//   dq = bf16(dq_acc)                                              (post-pass)
// --------------------------------------------------------------------------------------------
struct BwdParams {
  const bf16 *q, *k, *v, *o, *dout;
  const float* lse;
  float *delta, *dq_acc;
  bf16 *dq, *dk, *dv;
  int B, Sq, Sk, hq, hkv;
  long long q_ts, k_ts, v_ts, o_ts, do_ts, dq_ts, dk_ts, dv_ts;
  float scale;
  int causal;
};

template <int D>
__global__ void flash_delta_kernel(const BwdParams p) {
  const int lane = threadIdx.x & 31;
  const long long total = (long long)p.B * p.Sq * p.hq;
  for (long long idx = (long long)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5); idx < total;
       idx += (long long)gridDim.x * (blockDim.x >> 5)) {
    const int h = (int)(idx % p.hq);
    const long long bi = idx / p.hq;  // b * Sq + i
    const bf16* o = p.o + bi * p.o_ts + (long long)h * D;
    const bf16* d = p.dout + bi * p.do_ts + (long long)h * D;
    float s = 0.f;
    for (int c = lane * 2; c < D; c += 64) {
      const float2 a = __bfloat1622float2(*reinterpret_cast<const bf162*>(o + c));
      const float2 e = __bfloat1622float2(*reinterpret_cast<const bf162*>(d + c));
      s += a.x * e.x + a.y * e.y;
    }
    s = warp_sum(s);
    if (lane == 0) {
      const int b = (int)(bi / p.Sq), i = (int)(bi % p.Sq);
      p.delta[((long long)b * p.hq + h) * p.Sq + i] = s;
    }
  }
}

template <int D>
__global__ void __launch_bounds__(128, 1) flash_bwd_kernel(const BwdParams p) {
  constexpr int BM = 64, BN = 64, NT = 128, LDS = D + 8, LDP = BM + 8;
  extern __shared__ __align__(16) uint8_t smem_raw[];
  bf16* sK = reinterpret_cast<bf16*>(smem_raw);   // [BN][LDS]
  bf16* sV = sK + BN * LDS;                       // [BN][LDS]
  bf16* sQ = sV + BN * LDS;                       // [2][BM][LDS]
  bf16* sdO = sQ + 2 * BM * LDS;                  // [2][BM][LDS]
  bf16* sdS = sdO + 2 * BM * LDS;                 // [BN][LDP]  dS^T, rows = keys
  float* sLse = reinterpret_cast<float*>(sdS + BN * LDP);  // [2][BM]
  float* sDelta = sLse + 2 * BM;                           // [2][BM]

  const int nb = blockIdx.x, hk = blockIdx.y, b = blockIdx.z;
  const int n0 = nb * BN;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int g = lane >> 2, t = lane & 3;
  const int off = p.Sk - p.Sq;
  const int rep = p.hq / p.hkv;
  const float sl2 = p.scale * 1.4426950408889634f;
  const float l2e = 1.4426950408889634f;

  const bf16* kg = p.k + ((long long)b * p.Sk + n0) * p.k_ts + (long long)hk * D;
  const bf16* vg = p.v + ((long long)b * p.Sk + n0) * p.v_ts + (long long)hk * D;
  load_tile<BN, D, LDS, NT>(sK, kg, p.k_ts, p.Sk - n0);
  load_tile<BN, D, LDS, NT>(sV, vg, p.v_ts, p.Sk - n0);
  cp_async_commit();

  const int n_mblocks = (p.Sq + BM - 1) / BM;
  int mb_first = 0;
  if (p.causal) {
    const int first_row = n0 - off;  // first query that sees key n0
    mb_first = first_row > 0 ? first_row / BM : 0;
  }
  const int per_head = n_mblocks > mb_first ? n_mblocks - mb_first : 0;
  const int total_it = per_head * rep;

  auto issue_loads = [&](int it, int buf) {
    const int h = hk * rep + it / per_head;
    const int mb = mb_first + it % per_head;
    const int m0 = mb * BM;
    const bf16* qg = p.q + ((long long)b * p.Sq + m0) * p.q_ts + (long long)h * D;
    const bf16* dg = p.dout + ((long long)b * p.Sq + m0) * p.do_ts + (long long)h * D;
    load_tile<BM, D, LDS, NT>(sQ + buf * BM * LDS, qg, p.q_ts, p.Sq - m0);
    load_tile<BM, D, LDS, NT>(sdO + buf * BM * LDS, dg, p.do_ts, p.Sq - m0);
    if (threadIdx.x < BM) {
      const int i = m0 + threadIdx.x;
      const long long li = ((long long)b * p.hq + h) * p.Sq + i;
      sLse[buf * BM + threadIdx.x] = (i < p.Sq) ? p.lse[li] : INFINITY;   // +inf => P = 0 for padded rows
      sDelta[buf * BM + threadIdx.x] = (i < p.Sq) ? p.delta[li] : 0.f;
    }
  };

  float dk_acc[D / 8][4], dv_acc[D / 8][4];
#pragma unroll
  for (int i = 0; i < D / 8; i++) {
    dk_acc[i][0] = dk_acc[i][1] = dk_acc[i][2] = dk_acc[i][3] = 0.f;
    dv_acc[i][0] = dv_acc[i][1] = dv_acc[i][2] = dv_acc[i][3] = 0.f;
  }

  if (total_it > 0) {
    issue_loads(0, 0);
    cp_async_commit();
  }

  for (int it = 0; it < total_it; it++) {
    const int buf = it & 1;
    const int h = hk * rep + it / per_head;
    const int mb = mb_first + it % per_head;
    const int m0 = mb * BM;
    cp_async_wait<0>();
    __syncthreads();   // Q/dO[buf] (and K/V) landed; everyone is done with buffer buf^1 and with sdS
    if (it + 1 < total_it) {
      issue_loads(it + 1, buf ^ 1);
      cp_async_commit();
    }
    const bf16* sQb = sQ + buf * BM * LDS;
    const bf16* sdOb = sdO + buf * BM * LDS;
    const float* lse_b = sLse + buf * BM;
    const float* del_b = sDelta + buf * BM;

    // S^T[key, query] = K Q^T  (this warp: 16 key rows)
    float st[BM / 8][4];
#pragma unroll
    for (int i = 0; i < BM / 8; i++) st[i][0] = st[i][1] = st[i][2] = st[i][3] = 0.f;
#pragma unroll
    for (int kk = 0; kk < D / 16; kk++) {
      uint32_t a[4];
      {
        const int r = warp * 16 + (lane & 7) + ((lane >> 3) & 1) * 8;
        const int c = kk * 16 + (lane >> 4) * 8;
        ldsm_x4(smem_u32(sK + r * LDS + c), a[0], a[1], a[2], a[3]);
      }
#pragma unroll
      for (int nt = 0; nt < BM / 16; nt++) {
        uint32_t b0, b1, b2, b3;
        const int n = nt * 16 + (lane & 7) + (lane >> 4) * 8;
        const int c = kk * 16 + ((lane >> 3) & 1) * 8;
        ldsm_x4(smem_u32(sQb + n * LDS + c), b0, b1, b2, b3);
        mma16816(st[2 * nt], a, b0, b1);
        mma16816(st[2 * nt + 1], a, b2, b3);
      }
    }
    // P^T = exp(scale * S^T - lse[query]); masked / out-of-range -> 0
    const int key0 = n0 + warp * 16 + g;
#pragma unroll
    for (int i = 0; i < BM / 8; i++) {
#pragma unroll
      for (int e = 0; e < 4; e++) {
        const int qi = i * 8 + 2 * t + (e & 1);      // query index inside the block
        const int key = key0 + (e >> 1) * 8;
        const float l = lse_b[qi];
        float pv = exp2f(st[i][e] * sl2 - l * l2e);
        if (key >= p.Sk || (p.causal && key > m0 + qi + off) || l == INFINITY) pv = 0.f;
        st[i][e] = pv;
      }
    }
    // dV += P^T dO   (A = P^T from registers, B = dO [query][d] via transposed ldmatrix)
    uint32_t pt[BM / 16][4];
#pragma unroll
    for (int kb = 0; kb < BM / 16; kb++) {
      pt[kb][0] = pack_bf16(st[2 * kb][0], st[2 * kb][1]);
      pt[kb][1] = pack_bf16(st[2 * kb][2], st[2 * kb][3]);
      pt[kb][2] = pack_bf16(st[2 * kb + 1][0], st[2 * kb + 1][1]);
      pt[kb][3] = pack_bf16(st[2 * kb + 1][2], st[2 * kb + 1][3]);
    }
#pragma unroll
    for (int kb = 0; kb < BM / 16; kb++) {
#pragma unroll
      for (int dt = 0; dt < D / 16; dt++) {
        uint32_t b0, b1, b2, b3;
        const int kr = kb * 16 + (lane & 7) + ((lane >> 3) & 1) * 8;
        const int c = dt * 16 + (lane >> 4) * 8;
        ldsm_x4_t(smem_u32(sdOb + kr * LDS + c), b0, b1, b2, b3);
        mma16816(dv_acc[2 * dt], pt[kb], b0, b1);
        mma16816(dv_acc[2 * dt + 1], pt[kb], b2, b3);
      }
    }
    // dP^T[key, query] = V dO^T
    float dp[BM / 8][4];
#pragma unroll
    for (int i = 0; i < BM / 8; i++) dp[i][0] = dp[i][1] = dp[i][2] = dp[i][3] = 0.f;
#pragma unroll
    for (int kk = 0; kk < D / 16; kk++) {
      uint32_t a[4];
      {
        const int r = warp * 16 + (lane & 7) + ((lane >> 3) & 1) * 8;
        const int c = kk * 16 + (lane >> 4) * 8;
        ldsm_x4(smem_u32(sV + r * LDS + c), a[0], a[1], a[2], a[3]);
      }
#pragma unroll
      for (int nt = 0; nt < BM / 16; nt++) {
        uint32_t b0, b1, b2, b3;
        const int n = nt * 16 + (lane & 7) + (lane >> 4) * 8;
        const int c = kk * 16 + ((lane >> 3) & 1) * 8;
        ldsm_x4(smem_u32(sdOb + n * LDS + c), b0, b1, b2, b3);
        mma16816(dp[2 * nt], a, b0, b1);
        mma16816(dp[2 * nt + 1], a, b2, b3);
      }
    }
    // dS^T = P^T (dP^T - delta) * scale -> registers (A operand for dK) and smem (for dQ)
    uint32_t ds[BM / 16][4];
#pragma unroll
    for (int i = 0; i < BM / 8; i++) {
      const int qa = i * 8 + 2 * t;
      const float d0 = del_b[qa], d1 = del_b[qa + 1];
      dp[i][0] = st[i][0] * (dp[i][0] - d0) * p.scale;
      dp[i][1] = st[i][1] * (dp[i][1] - d1) * p.scale;
      dp[i][2] = st[i][2] * (dp[i][2] - d0) * p.scale;
      dp[i][3] = st[i][3] * (dp[i][3] - d1) * p.scale;
      const uint32_t lo = pack_bf16(dp[i][0], dp[i][1]);
      const uint32_t hi = pack_bf16(dp[i][2], dp[i][3]);
      *reinterpret_cast<uint32_t*>(sdS + (warp * 16 + g) * LDP + qa) = lo;
      *reinterpret_cast<uint32_t*>(sdS + (warp * 16 + g + 8) * LDP + qa) = hi;
      ds[i >> 1][(i & 1) * 2] = lo;
      ds[i >> 1][(i & 1) * 2 + 1] = hi;
    }
    // dK += dS^T Q   (B = Q [query][d] via transposed ldmatrix)
#pragma unroll
    for (int kb = 0; kb < BM / 16; kb++) {
#pragma unroll
      for (int dt = 0; dt < D / 16; dt++) {
        uint32_t b0, b1, b2, b3;
        const int kr = kb * 16 + (lane & 7) + ((lane >> 3) & 1) * 8;
        const int c = dt * 16 + (lane >> 4) * 8;
        ldsm_x4_t(smem_u32(sQb + kr * LDS + c), b0, b1, b2, b3);
        mma16816(dk_acc[2 * dt], ds[kb], b0, b1);
        mma16816(dk_acc[2 * dt + 1], ds[kb], b2, b3);
      }
    }
    __syncthreads();  // dS^T of all four warps is in smem
    // dQ[query, d] += dS[query, key] K[key, d]   (this warp: 16 query rows; A = dS^T transposed on load)
    {
      float dq[D / 8][4];
#pragma unroll
      for (int i = 0; i < D / 8; i++) dq[i][0] = dq[i][1] = dq[i][2] = dq[i][3] = 0.f;
#pragma unroll
      for (int kb = 0; kb < BN / 16; kb++) {
        uint32_t a[4];
        {
          const int kr = kb * 16 + (lane & 7) + (lane >> 4) * 8;          // stored row = key
          const int mc = warp * 16 + ((lane >> 3) & 1) * 8;               // stored col = query
          ldsm_x4_t(smem_u32(sdS + kr * LDP + mc), a[0], a[1], a[2], a[3]);
        }
#pragma unroll
        for (int dt = 0; dt < D / 16; dt++) {
          uint32_t b0, b1, b2, b3;
          const int kr = kb * 16 + (lane & 7) + ((lane >> 3) & 1) * 8;
          const int c = dt * 16 + (lane >> 4) * 8;
          ldsm_x4_t(smem_u32(sK + kr * LDS + c), b0, b1, b2, b3);
          mma16816(dq[2 * dt], a, b0, b1);
          mma16816(dq[2 * dt + 1], a, b2, b3);
        }
      }
      const int qrow = m0 + warp * 16 + g;
      float* dst = p.dq_acc + (((long long)b * p.Sq + qrow) * p.hq + h) * D + 2 * t;
#pragma unroll
      for (int i = 0; i < D / 8; i++) {
        if (qrow < p.Sq) atomicAdd(reinterpret_cast<float2*>(dst + i * 8), make_float2(dq[i][0], dq[i][1]));
        if (qrow + 8 < p.Sq)
          atomicAdd(reinterpret_cast<float2*>(dst + (long long)8 * p.hq * D + i * 8), make_float2(dq[i][2], dq[i][3]));
      }
    }
  }
  cp_async_wait<0>();
  __syncthreads();

  // write dK, dV (stage through sQ / sdO regions for 16-byte stores)
  bf16* sOutK = sQ;
  bf16* sOutV = sdO;
#pragma unroll
  for (int i = 0; i < D / 8; i++) {
    const int c = i * 8 + 2 * t;
    *reinterpret_cast<uint32_t*>(sOutK + (warp * 16 + g) * LDS + c) = pack_bf16(dk_acc[i][0], dk_acc[i][1]);
    *reinterpret_cast<uint32_t*>(sOutK + (warp * 16 + g + 8) * LDS + c) = pack_bf16(dk_acc[i][2], dk_acc[i][3]);
    *reinterpret_cast<uint32_t*>(sOutV + (warp * 16 + g) * LDS + c) = pack_bf16(dv_acc[i][0], dv_acc[i][1]);
    *reinterpret_cast<uint32_t*>(sOutV + (warp * 16 + g + 8) * LDS + c) = pack_bf16(dv_acc[i][2], dv_acc[i][3]);
  }
  __syncthreads();
  bf16* dkg = p.dk + ((long long)b * p.Sk + n0) * p.dk_ts + (long long)hk * D;
  bf16* dvg = p.dv + ((long long)b * p.Sk + n0) * p.dv_ts + (long long)hk * D;
  constexpr int VPR = D / 8;
  for (int i = threadIdx.x; i < BN * VPR; i += NT) {
    const int r = i / VPR, c = i % VPR;
    if (n0 + r < p.Sk) {
      *reinterpret_cast<uint4*>(dkg + (long long)r * p.dk_ts + c * 8) = *reinterpret_cast<const uint4*>(sOutK + r * LDS + c * 8);
      *reinterpret_cast<uint4*>(dvg + (long long)r * p.dv_ts + c * 8) = *reinterpret_cast<const uint4*>(sOutV + r * LDS + c * 8);
    }
  }
}

template <int D>
__global__ void flash_dq_convert_kernel(const BwdParams p) {
  constexpr int VPR = D / 8;
  const long long total = (long long)p.B * p.Sq * p.hq * VPR;
  for (long long idx = (long long)blockIdx.x * blockDim.x + threadIdx.x; idx < total;
       idx += (long long)gridDim.x * blockDim.x) {
    const int v = (int)(idx % VPR);
    const long long th = idx / VPR;
    const int h = (int)(th % p.hq);
    const long long bi = th / p.hq;
    const float4* src = reinterpret_cast<const float4*>(p.dq_acc + (bi * p.hq + h) * D + v * 8);
    const float4 a = src[0], c = src[1];
    const float f[8] = {a.x, a.y, a.z, a.w, c.x, c.y, c.z, c.w};
    *reinterpret_cast<uint4*>(p.dq + bi * p.dq_ts + (long long)h * D + v * 8) = pack8(f);
  }
}

template <int D>
int launch_fwd(const FwdParams& p, cudaStream_t s) {
  constexpr int LDS = D + 8;
  const int smem = (128 + 4 * 64) * LDS * 2;
  static bool attr = false;
  if (!attr) {
    cudaFuncSetAttribute(flash_fwd_kernel<D>, cudaFuncAttributeMaxDynamicSharedMemorySize, smem);
    attr = true;
  }
  dim3 grid((p.Sq + 127) / 128, p.hq, p.B);
  flash_fwd_kernel<D><<<grid, 256, smem, s>>>(p);
  LB_CHECK_LAUNCH();
  return LB_OK;
}

template <int D>
int launch_bwd(const BwdParams& p, cudaStream_t s) {
  constexpr int LDS = D + 8;
  const int smem = (2 * 64 + 4 * 64) * LDS * 2 + 64 * (64 + 8) * 2 + 4 * 64 * 4;
  static bool attr = false;
  if (!attr) {
    cudaFuncSetAttribute(flash_bwd_kernel<D>, cudaFuncAttributeMaxDynamicSharedMemorySize, smem);
    attr = true;
  }
  const long long rows = (long long)p.B * p.Sq * p.hq;
  int dblocks = (int)((rows + 7) / 8 > lb_num_sms() * 8 ? lb_num_sms() * 8 : (rows + 7) / 8);
  flash_delta_kernel<D><<<dblocks, 256, 0, s>>>(p);
  LB_CHECK_LAUNCH();
  dim3 grid((p.Sk + 63) / 64, p.hkv, p.B);
  flash_bwd_kernel<D><<<grid, 128, smem, s>>>(p);
  LB_CHECK_LAUNCH();
  const long long total = rows * (D / 8);
  int cblocks = (int)((total + 255) / 256 > lb_num_sms() * 16 ? lb_num_sms() * 16 : (total + 255) / 256);
  flash_dq_convert_kernel<D><<<cblocks, 256, 0, s>>>(p);
  LB_CHECK_LAUNCH();
  return LB_OK;
}

}  // namespace

extern "C" int lb_flash_fwd(const void* q, const void* k, const void* v, void* o, void* lse, int B, int Sq, int Sk,
                            int hq, int hkv, int d, long long q_ts, long long k_ts, long long v_ts, long long o_ts,
                            float scale, int causal, void* stream) {
  if (B <= 0 || Sq <= 0 || Sk <= 0 || hq % hkv) return LB_ERR_SHAPE;
  if ((q_ts | k_ts | v_ts | o_ts) % 8) return LB_ERR_SHAPE;
  FwdParams p{(const bf16*)q, (const bf16*)k, (const bf16*)v, (bf16*)o, (float*)lse, B, Sq, Sk, hq, hkv,
              q_ts, k_ts, v_ts, o_ts, scale, causal};
  cudaStream_t s = (cudaStream_t)stream;
  switch (d) {
    case 32: return launch_fwd<32>(p, s);
    case 64: return launch_fwd<64>(p, s);
    case 128: return launch_fwd<128>(p, s);
    default: return LB_ERR_SHAPE;
  }
}

// dq_acc: zero-initialised fp32 scratch [B, Sq, hq, d]; delta: fp32 scratch [B, hq, Sq].
extern "C" int lb_flash_bwd(const void* q, const void* k, const void* v, const void* o, const void* dout,
                            const void* lse, void* delta, void* dq_acc, void* dq, void* dk, void* dv, int B, int Sq,
                            int Sk, int hq, int hkv, int d, long long q_ts, long long k_ts, long long v_ts,
                            long long o_ts, long long do_ts, long long dq_ts, long long dk_ts, long long dv_ts,
                            float scale, int causal, void* stream) {
  if (B <= 0 || Sq <= 0 || Sk <= 0 || hq % hkv) return LB_ERR_SHAPE;
  if ((q_ts | k_ts | v_ts | o_ts | do_ts | dq_ts | dk_ts | dv_ts) % 8) return LB_ERR_SHAPE;
  BwdParams p{(const bf16*)q, (const bf16*)k, (const bf16*)v, (const bf16*)o, (const bf16*)dout, (const float*)lse,
              (float*)delta, (float*)dq_acc, (bf16*)dq, (bf16*)dk, (bf16*)dv, B, Sq, Sk, hq, hkv,
              q_ts, k_ts, v_ts, o_ts, do_ts, dq_ts, dk_ts, dv_ts, scale, causal};
  cudaStream_t s = (cudaStream_t)stream;
  switch (d) {
    case 32: return launch_bwd<32>(p, s);
    case 64: return launch_bwd<64>(p, s);
    case 128: return launch_bwd<128>(p, s);
    default: return LB_ERR_SHAPE;
  }
}
