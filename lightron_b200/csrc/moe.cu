// Mixture-of-experts routing and expert-parallel token exchange over NVLink peer memory.
//
// What the reference does with library calls and host round trips (softmax / topk,
// parallel/parallel_ep.py: argsort, bincount, a count all-to-all whose result is read on the host,
// a variable-size all-to-all, index_copy_, a weighted sum) is done here by five kernels, none of
// which returns anything to the host:
//
//   moe_router_kernel    gate GEMM (E is tiny: one warp per token, fp32 dot products), softmax,
//                        top-k, and for every (token, slot) copy its rank among the copies of the
//                        same expert inside the same 32-token block, plus per-block histograms
//   moe_plan_kernel      one CTA: prefix sums over the blocks, this rank's per-expert counts stored
//                        into every peer's count table (flag per source rank), then, from the full
//                        [ranks x experts] table, the row in the owner's buffer where this rank's
//                        copies of every expert start, the layout of the local expert segments
//                        (each starts on a multiple of 128 rows) and the load-balance loss
//   moe_push_kernel      dispatch (and the backward of combine): every copy's row is stored, scaled
//                        if asked, straight into the expert owner's buffer with 16-byte peer stores;
//                        every CTA counts itself in each destination's arrival word when its stores
//                        are fenced; the owner zeroes the padding rows of its segments
//   moe_pull_kernel      combine (and the backward of dispatch): a token's k expert outputs are read
//                        from their owners with 16-byte peer loads, weighted and summed; the same
//                        pass can produce the dot products that are the router-weight gradients
//   moe_router_bwd_kernel  softmax backward, dx = dlogits . Wg, dWg += dlogits^T x
//
// The grouped expert GEMM between push and pull (lb_gemm_ragged, gemm_grouped.cu) takes the segment
// offsets and counts from device memory and waits for the arrival word itself.
//
// All waits on a peer are bounded (comm.cuh) and report through lb_moe_status(); row indices are
// checked against the buffer capacity before every store or load (a routing so skewed that a rank
// would receive more than its capacity sets the status word instead of writing out of bounds).
#include "comm.cuh"

static __device__ unsigned int g_moe_status[4] = {0, 0, 0, 0};

namespace {

constexpr int MOE_MAX_RANKS = 8;
constexpr int MOE_MAX_EXPERTS = 64;
constexpr int MOE_MAX_TOPK = 8;
constexpr int ROUTER_TOKENS = 32;       // tokens per router block (the unit of the within-block ranks)
constexpr int ROUTER_THREADS = 256;

// A copy routed to a row beyond the expert-side capacity is DROPPED (not dispatched, contributes
// nothing to the combine), as in capacity-factor routing; it is counted, not treated as a failure:
// word 2 = dropped copies / overfull plans since the last read, word 3 = largest row count asked for.
__device__ __forceinline__ void moe_overflow(unsigned rows_wanted) {
  atomicAdd(&g_moe_status[2], 1u);
  atomicMax(&g_moe_status[3], rows_wanted);
}
__device__ __forceinline__ void moe_fail(unsigned code, unsigned where) {
  if (atomicCAS(&g_moe_status[0], 0u, code) == 0u) atomicExch(&g_moe_status[1], where);
}

// -------------------------------------------------------------------------------------------
// Router
// -------------------------------------------------------------------------------------------
__global__ void __launch_bounds__(ROUTER_THREADS)
moe_router_kernel(const bf16* __restrict__ x, const bf16* __restrict__ wg, int T, int H, int E, int k,
                  float* __restrict__ probs, int* __restrict__ idx, float* __restrict__ wts, int* __restrict__ within,
                  int* __restrict__ blk_hist, float* __restrict__ blk_psum) {
  __shared__ int s_eid[ROUTER_TOKENS * MOE_MAX_TOPK];
  __shared__ int s_hist[MOE_MAX_EXPERTS];
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int t0 = blockIdx.x * ROUTER_TOKENS;
  for (int i = threadIdx.x; i < MOE_MAX_EXPERTS; i += blockDim.x) s_hist[i] = 0;
  for (int i = threadIdx.x; i < ROUTER_TOKENS * MOE_MAX_TOPK; i += blockDim.x) s_eid[i] = -1;
  __syncthreads();
  const int nvec = H >> 3;
  for (int tl = warp; tl < ROUTER_TOKENS; tl += ROUTER_THREADS / 32) {
    const int t = t0 + tl;
    if (t >= T) break;                                   // warp-uniform
    const uint4* xr = reinterpret_cast<const uint4*>(x + (size_t)t * H);
    // logits[e] for e = lane, lane + 32 end up in lg0 / lg1 (E <= 64)
    float lg0 = -INFINITY, lg1 = -INFINITY;
    for (int e0 = 0; e0 < E; e0 += 8) {                   // 8 experts per pass over the row
      float acc[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
      const int ne = min(8, E - e0);
      for (int v = lane; v < nvec; v += 32) {
        float xf[8];
        unpack8(xr[v], xf);
#pragma unroll
        for (int j = 0; j < 8; j++) {
          if (j < ne) {
            float wf[8];
            unpack8(__ldg(reinterpret_cast<const uint4*>(wg + (size_t)(e0 + j) * H) + v), wf);
#pragma unroll
            for (int i = 0; i < 8; i++) acc[j] = fmaf(xf[i], wf[i], acc[j]);
          }
        }
      }
#pragma unroll
      for (int j = 0; j < 8; j++) {
        const float s = warp_sum(acc[j]);
        if (j < ne) {
          const int e = e0 + j;
          if ((e & 31) == lane) { if (e < 32) lg0 = s; else lg1 = s; }
        }
      }
    }
    // softmax over experts (fp32), every lane ends with its own probabilities
    const float mx = warp_max(fmaxf(lg0, lg1));
    const float ex0 = (lane < E) ? __expf(lg0 - mx) : 0.f;
    const float ex1 = (lane + 32 < E) ? __expf(lg1 - mx) : 0.f;
    const float inv = 1.f / warp_sum(ex0 + ex1);
    const float p0 = ex0 * inv, p1 = ex1 * inv;
    if (lane < E) probs[(size_t)t * E + lane] = p0;
    if (lane + 32 < E) probs[(size_t)t * E + lane + 32] = p1;
    // top-k: k rounds of arg-max (lowest index wins ties)
    float q0 = (lane < E) ? p0 : -1.f, q1 = (lane + 32 < E) ? p1 : -1.f;
    for (int s = 0; s < k; s++) {
      float best = fmaxf(q0, q1);
      int bi = (q0 >= q1) ? lane : lane + 32;
#pragma unroll
      for (int o = 16; o > 0; o >>= 1) {
        const float ob = __shfl_xor_sync(0xffffffffu, best, o);
        const int oi = __shfl_xor_sync(0xffffffffu, bi, o);
        if (ob > best || (ob == best && oi < bi)) { best = ob; bi = oi; }
      }
      if (lane == 0) {
        idx[(size_t)t * k + s] = bi;
        wts[(size_t)t * k + s] = best;
        s_eid[tl * k + s] = bi;
      }
      if (bi == lane) q0 = -1.f;
      if (bi == lane + 32) q1 = -1.f;
    }
  }
  __syncthreads();
  // rank of every copy among the block's earlier copies of the same expert, in (token, slot) order
  const int ncopies = ROUTER_TOKENS * k;
  for (int c = threadIdx.x; c < ncopies; c += blockDim.x) {
    const int e = s_eid[c];
    if (e < 0) continue;
    int r = 0;
    for (int j = 0; j < c; j++) r += (s_eid[j] == e);
    within[(size_t)t0 * k + c] = r;
    atomicAdd(&s_hist[e], 1);
  }
  __syncthreads();
  for (int e = threadIdx.x; e < E; e += blockDim.x) {
    // probability mass per expert over the block's tokens, summed in token order (deterministic)
    float ps = 0.f;
    for (int tl = 0; tl < ROUTER_TOKENS && t0 + tl < T; tl++) ps += probs[(size_t)(t0 + tl) * E + e];
    blk_hist[(size_t)blockIdx.x * E + e] = s_hist[e];
    blk_psum[(size_t)blockIdx.x * E + e] = ps;
  }
}

// -------------------------------------------------------------------------------------------
// Plan
// -------------------------------------------------------------------------------------------
struct PlanParams {
  const int* blk_hist;      // [nblk, E]
  const float* blk_psum;    // [nblk, E]
  int* blk_base;            // [nblk, E] out: copies of expert e in earlier blocks of this rank
  int* dst_row0;            // [E] out: row in the owner's buffer where this rank's copies of e start
  int* seg;                 // [2 * LE + 2] out: offsets[LE], counts[LE], padded end, total received
  float* frac;              // [E] out: fraction of this rank's copies routed to e
  float* aux;               // [1] out: load-balance loss E * sum_e frac_e * mean_t p_te
  int nblk, E, LE, n, me, T, k, cap;
  int* cnt_all[MOE_MAX_RANKS];          // rank r's count table [2][n][E]
  unsigned int* flags[MOE_MAX_RANKS];   // rank r's "counts arrived" words [n]
  int parity;
  unsigned int epoch;
  unsigned long long wait_ns;
};

__global__ void __launch_bounds__(256) moe_plan_kernel(const PlanParams p) {
  __shared__ int s_cnt[MOE_MAX_EXPERTS];
  __shared__ float s_ps[MOE_MAX_EXPERTS];
  __shared__ int s_all[MOE_MAX_RANKS * MOE_MAX_EXPERTS];
  __shared__ int s_fail;
  const int tid = threadIdx.x;
  if (tid == 0) s_fail = 0;
  if (tid < p.E) {
    int run = 0;
    float ps = 0.f;
    for (int b = 0; b < p.nblk; b++) {
      p.blk_base[(size_t)b * p.E + tid] = run;
      run += p.blk_hist[(size_t)b * p.E + tid];
      ps += p.blk_psum[(size_t)b * p.E + tid];
    }
    s_cnt[tid] = run;
    s_ps[tid] = ps;
    p.frac[tid] = (float)run / (float)((long long)p.T * p.k);
    for (int r = 0; r < p.n; r++) p.cnt_all[r][((size_t)p.parity * p.n + p.me) * p.E + tid] = run;
  }
  __syncthreads();
  if (tid < p.n) {
    __threadfence_system();
    lbcomm::st_release_sys(p.flags[tid] + p.me, p.epoch);
    if (!lbcomm::flag_wait_ge(p.flags[p.me] + tid, p.epoch, p.wait_ns)) { s_fail = 1; moe_fail(1u, 1u); }
  }
  __syncthreads();
  if (s_fail) return;
  const volatile int* mine = p.cnt_all[p.me] + (size_t)p.parity * p.n * p.E;
  for (int i = tid; i < p.n * p.E; i += blockDim.x) s_all[i] = mine[i];
  __syncthreads();
  if (tid < p.E) {
    const int d = tid / p.LE, le = tid - d * p.LE;
    int base = 0;
    for (int j = 0; j < le; j++) {          // padded sizes of the owner's earlier local experts
      int tot = 0;
      for (int s = 0; s < p.n; s++) tot += s_all[s * p.E + d * p.LE + j];
      base += (tot + 127) & ~127;
    }
    int before = 0, tot = 0;
    for (int s = 0; s < p.n; s++) {
      const int c = s_all[s * p.E + tid];
      if (s < p.me) before += c;
      tot += c;
    }
    p.dst_row0[tid] = base + before;
    if (d == p.me) {
      p.seg[le] = base;
      p.seg[p.LE + le] = tot;
      if (le == p.LE - 1) {
        const int end = base + ((tot + 127) & ~127);
        p.seg[2 * p.LE] = end;
        if (end > p.cap) moe_overflow((unsigned)end);        // more rows routed here than the buffers hold: the excess is dropped
      }
    }
  }
  if (tid == 0) {
    int total = 0;
    for (int le = 0; le < p.LE; le++)
      for (int s = 0; s < p.n; s++) total += s_all[s * p.E + p.me * p.LE + le];
    p.seg[2 * p.LE + 1] = total;
    float a = 0.f;
    for (int e = 0; e < p.E; e++) a += ((float)s_cnt[e] / (float)((long long)p.T * p.k)) * (s_ps[e] / (float)p.T);
    p.aux[0] = a * (float)p.E;
  }
}

// -------------------------------------------------------------------------------------------
// Push: dst_owner[row(t, s)] = scale[t, s] * src[t]
// -------------------------------------------------------------------------------------------
struct PushParams {
  const bf16* src;          // [T, H]
  const float* scale;       // [T, k] or null
  const int* idx;           // [T, k] expert of every copy
  const int* within;        // [T, k]   (compute_rows)
  const int* blk_base;      // [nblk, E] (compute_rows)
  const int* dst_row0;      // [E]       (compute_rows)
  int* rows;                // [T, k]: written when compute_rows, read otherwise
  const int* seg;           // local segment table (for zeroing the padding rows of `own`)
  bf16* own;                // this rank's buffer (== dst[me])
  bf16* dst[MOE_MAX_RANKS];
  unsigned int* arrive[MOE_MAX_RANKS];   // rank r's arrival word for this buffer
  int T, H, E, LE, k, n, me, cap, compute_rows;
};

__global__ void __launch_bounds__(256) moe_push_kernel(const PushParams p) {
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, wpb = blockDim.x >> 5;
  const int nvec = p.H >> 3;
  // padding rows of the local segments: rows [off + cnt, off + round_up(cnt, 128)) become zero
  for (int le = 0; le < p.LE; le++) {
    const int off = p.seg[le], cnt = p.seg[p.LE + le];
    const int pad0 = off + cnt, pad1 = min(off + ((cnt + 127) & ~127), p.cap);
    for (int r = pad0 + blockIdx.x * wpb + warp; r < pad1; r += gridDim.x * wpb) {
      uint4* d = reinterpret_cast<uint4*>(p.own + (size_t)r * p.H);
      for (int v = lane; v < nvec; v += 32) d[v] = make_uint4(0, 0, 0, 0);
    }
  }
  for (int t = blockIdx.x * wpb + warp; t < p.T; t += gridDim.x * wpb) {
    const uint4* sr = reinterpret_cast<const uint4*>(p.src + (size_t)t * p.H);
    uint4* drow[MOE_MAX_TOPK];
    float sc[MOE_MAX_TOPK];
#pragma unroll
    for (int s = 0; s < MOE_MAX_TOPK; s++) {
      drow[s] = nullptr;
      sc[s] = 1.f;
      if (s < p.k) {
        const int e = p.idx[(size_t)t * p.k + s];
        const bool e_ok = e >= 0 && e < p.E;
        int row = -1;
        if (p.compute_rows) {
          if (e_ok) row = p.dst_row0[e] + p.blk_base[(size_t)(t / ROUTER_TOKENS) * p.E + e] + p.within[(size_t)t * p.k + s];
          if (lane == 0) p.rows[(size_t)t * p.k + s] = row;
        } else {
          row = p.rows[(size_t)t * p.k + s];
        }
        if (e_ok && row >= 0 && row < p.cap) drow[s] = reinterpret_cast<uint4*>(p.dst[e / p.LE] + (size_t)row * p.H);
        else if (lane == 0) { if (e_ok && row >= p.cap) moe_overflow((unsigned)row + 1u); else moe_fail(4u, (unsigned)row); }
        if (p.scale) sc[s] = p.scale[(size_t)t * p.k + s];
      }
    }
    for (int v = lane; v < nvec; v += 32) {
      const uint4 raw = sr[v];
      if (p.scale) {
        float f[8];
        unpack8(raw, f);
#pragma unroll
        for (int s = 0; s < MOE_MAX_TOPK; s++) {
          if (s < p.k && drow[s]) {
            float g[8];
#pragma unroll
            for (int i = 0; i < 8; i++) g[i] = f[i] * sc[s];
            drow[s][v] = pack8(g);
          }
        }
      } else {
#pragma unroll
        for (int s = 0; s < MOE_MAX_TOPK; s++)
          if (s < p.k && drow[s]) drow[s][v] = raw;
      }
    }
  }
  // every store of this CTA is fenced, then the CTA counts itself at every destination
  __threadfence_system();
  __syncthreads();
  if (threadIdx.x < p.n) {
    __threadfence_system();
    lbcomm::red_release_sys_add(p.arrive[threadIdx.x], 1u);
  }
}

// -------------------------------------------------------------------------------------------
// Pull: out[t] = sum_s w[t, s] * src_owner[row(t, s)];  dots[t, s] = <src_owner[row(t, s)], dots_with[t]>
// -------------------------------------------------------------------------------------------
struct PullParams {
  bf16* out;                // [T, H] or null
  const float* w;           // [T, k] or null (weights 1)
  const int* idx;           // [T, k]
  const int* rows;          // [T, k]
  float* dots;              // [T, k] or null
  const bf16* dots_with;    // [T, H] (with dots)
  const bf16* src[MOE_MAX_RANKS];
  unsigned int* ready[MOE_MAX_RANKS];    // rank r's "source buffer of rank q is complete" words [n]
  unsigned int epoch;
  unsigned long long wait_ns;
  int T, H, E, LE, k, n, me, cap;
};

__global__ void __launch_bounds__(256) moe_pull_kernel(const PullParams p) {
  __shared__ int s_fail;
  if (threadIdx.x == 0) s_fail = 0;
  __syncthreads();
  // this kernel runs behind the kernel that produced this rank's source buffer: tell every peer,
  // then wait until every peer's buffer is complete too
  if (threadIdx.x < p.n) {
    if (blockIdx.x == 0) {
      __threadfence_system();
      lbcomm::st_release_sys(p.ready[threadIdx.x] + p.me, p.epoch);
    }
    if (!lbcomm::flag_wait_ge(p.ready[p.me] + threadIdx.x, p.epoch, p.wait_ns)) { s_fail = 1; moe_fail(2u, 2u); }
  }
  __syncthreads();
  if (s_fail) return;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, wpb = blockDim.x >> 5;
  const int nvec = p.H >> 3;
  for (int t = blockIdx.x * wpb + warp; t < p.T; t += gridDim.x * wpb) {
    const uint4* srow[MOE_MAX_TOPK];
    float wt[MOE_MAX_TOPK], dot[MOE_MAX_TOPK];
#pragma unroll
    for (int s = 0; s < MOE_MAX_TOPK; s++) {
      srow[s] = nullptr;
      wt[s] = 1.f;
      dot[s] = 0.f;
      if (s < p.k) {
        const int e = p.idx[(size_t)t * p.k + s];
        const int row = p.rows[(size_t)t * p.k + s];
        if (e >= 0 && e < p.E && row >= 0 && row < p.cap)
          srow[s] = reinterpret_cast<const uint4*>(p.src[e / p.LE] + (size_t)row * p.H);
        else if (lane == 0 && !(e >= 0 && e < p.E && row >= p.cap)) moe_fail(5u, (unsigned)row);   // beyond capacity: dropped at dispatch
        if (p.w) wt[s] = p.w[(size_t)t * p.k + s];
      }
    }
    const uint4* dw = p.dots ? reinterpret_cast<const uint4*>(p.dots_with + (size_t)t * p.H) : nullptr;
    uint4* orow = p.out ? reinterpret_cast<uint4*>(p.out + (size_t)t * p.H) : nullptr;
    for (int v = lane; v < nvec; v += 32) {
      float acc[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
      float g[8];
      if (dw) unpack8(dw[v], g);
#pragma unroll
      for (int s = 0; s < MOE_MAX_TOPK; s++) {
        if (s < p.k && srow[s]) {
          float f[8];
          unpack8(lbcomm::ld_nc_v4(srow[s] + v), f);
#pragma unroll
          for (int i = 0; i < 8; i++) acc[i] = fmaf(wt[s], f[i], acc[i]);
          if (dw) {
#pragma unroll
            for (int i = 0; i < 8; i++) dot[s] = fmaf(f[i], g[i], dot[s]);
          }
        }
      }
      if (orow) orow[v] = pack8(acc);
    }
    if (p.dots) {
#pragma unroll
      for (int s = 0; s < MOE_MAX_TOPK; s++) {
        if (s < p.k) {
          const float d = warp_sum(dot[s]);
          if (lane == 0) p.dots[(size_t)t * p.k + s] = d;
        }
      }
    }
  }
}

// -------------------------------------------------------------------------------------------
// Router backward
// -------------------------------------------------------------------------------------------
constexpr int RB_TOKENS = 64;

__global__ void __launch_bounds__(256)
moe_router_bwd_kernel(const bf16* __restrict__ x, const bf16* __restrict__ wg, const float* __restrict__ probs,
                      const int* __restrict__ idx, const float* __restrict__ dwts, const float* __restrict__ frac,
                      const float* __restrict__ daux, bf16* __restrict__ dx, float* __restrict__ dwg_acc, int T, int H,
                      int E, int k) {
  __shared__ float s_dl[RB_TOKENS][MOE_MAX_EXPERTS + 1];
  const int t0 = blockIdx.x * RB_TOKENS;
  const int ntok = min(RB_TOKENS, T - t0);
  const float aux_c = daux ? daux[0] * (float)E / (float)T : 0.f;
  // dlogit[t, e] = p (dp - sum_e' p dp) with dp = routed-weight gradient + load-balance term
  for (int i = threadIdx.x; i < ntok; i += blockDim.x) {
    const int t = t0 + i;
    float dot = 0.f;
    for (int e = 0; e < E; e++) {
      float dp = aux_c * frac[e];
      for (int s = 0; s < k; s++) if (idx[(size_t)t * k + s] == e) dp += dwts[(size_t)t * k + s];
      s_dl[i][e] = dp;
      dot += probs[(size_t)t * E + e] * dp;
    }
    for (int e = 0; e < E; e++) s_dl[i][e] = probs[(size_t)t * E + e] * (s_dl[i][e] - dot);
  }
  __syncthreads();
  // every thread owns 8-column vectors v = tid, tid + 256, ...
  const int nvec = H >> 3;
  for (int v = threadIdx.x; v < nvec; v += blockDim.x) {
    // dx[t, cols] = sum_e dlogit[t, e] wg[e, cols]
    for (int i = 0; i < ntok; i++) {
      float acc[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
      for (int e = 0; e < E; e++) {
        float wf[8];
        unpack8(__ldg(reinterpret_cast<const uint4*>(wg + (size_t)e * H) + v), wf);
        const float d = s_dl[i][e];
#pragma unroll
        for (int j = 0; j < 8; j++) acc[j] = fmaf(d, wf[j], acc[j]);
      }
      *reinterpret_cast<uint4*>(dx + (size_t)(t0 + i) * H + v * 8) = pack8(acc);
    }
    // dwg[e, cols] += sum_t dlogit[t, e] x[t, cols], four experts at a time
    for (int e0 = 0; e0 < E; e0 += 4) {
      float acc[4][8];
#pragma unroll
      for (int a = 0; a < 4; a++)
#pragma unroll
        for (int j = 0; j < 8; j++) acc[a][j] = 0.f;
      for (int i = 0; i < ntok; i++) {
        float xf[8];
        unpack8(*reinterpret_cast<const uint4*>(x + (size_t)(t0 + i) * H + v * 8), xf);
#pragma unroll
        for (int a = 0; a < 4; a++) {
          if (e0 + a < E) {
            const float d = s_dl[i][e0 + a];
#pragma unroll
            for (int j = 0; j < 8; j++) acc[a][j] = fmaf(d, xf[j], acc[a][j]);
          }
        }
      }
#pragma unroll
      for (int a = 0; a < 4; a++) {
        if (e0 + a < E) {
          float* dst = dwg_acc + (size_t)(e0 + a) * H + v * 8;
#pragma unroll
          for (int j = 0; j < 8; j++) atomicAdd(dst + j, acc[a][j]);
        }
      }
    }
  }
}

int moe_grid(int T) {
  int blocks = (T + 7) / 8;
  const int cap = lb_num_sms() * 4;
  if (blocks > cap) blocks = cap;
  return blocks < 1 ? 1 : blocks;
}

}  // namespace

extern "C" int lb_moe_status(void* out) {
  cudaError_t e = cudaMemcpyFromSymbol(out, g_moe_status, sizeof(unsigned int) * 4);
  if (e != cudaSuccess) { g_lb_last_cuda_error = (int)e; return LB_ERR_LAUNCH; }
  unsigned int zeros[4] = {0, 0, 0, 0};
  cudaMemcpyToSymbol(g_moe_status, zeros, sizeof(zeros));
  return LB_OK;
}

// Number of router blocks (rows of blk_hist / blk_psum / blk_base) for T tokens.
extern "C" int lb_moe_router_blocks(int T) { return (T + ROUTER_TOKENS - 1) / ROUTER_TOKENS; }

// Number of CTAs lb_moe_push launches for T tokens on this device: every destination's arrival word
// grows by this much per source rank and call.
extern "C" int lb_moe_push_ctas(int T) { return moe_grid(T); }

// x [T, H] bf16, wg [E, H] bf16 -> probs [T, E] fp32, idx [T, k] int32, wts [T, k] fp32 (softmax
// probabilities of the chosen experts), within [T, k] int32, blk_hist [nblk, E] int32,
// blk_psum [nblk, E] fp32.  E <= 64, k <= 8, H a multiple of 8.
extern "C" int lb_moe_router(const void* x, const void* wg, int T, int H, int E, int k, void* probs, void* idx, void* wts,
                             void* within, void* blk_hist, void* blk_psum, void* stream) {
  if (T <= 0 || (H % 8) || E < 1 || E > MOE_MAX_EXPERTS || k < 1 || k > MOE_MAX_TOPK || k > E) return LB_ERR_SHAPE;
  moe_router_kernel<<<lb_moe_router_blocks(T), ROUTER_THREADS, 0, (cudaStream_t)stream>>>(
      (const bf16*)x, (const bf16*)wg, T, H, E, k, (float*)probs, (int*)idx, (float*)wts, (int*)within, (int*)blk_hist,
      (float*)blk_psum);
  LB_CHECK_LAUNCH();
  return LB_OK;
}

// cnt_ptrs[r] / flag_ptrs[r]: rank r's count table [2][n][E] int32 and "counts arrived" words [n]
// (peer-visible, zeroed once); epoch grows by one per call, parity alternates.  seg has 2 * LE + 2
// ints: segment offsets, segment counts, padded end of the last segment, rows received.
extern "C" int lb_moe_plan(const void* blk_hist, const void* blk_psum, void* blk_base, void* dst_row0, void* seg,
                           void* frac, void* aux, int nblk, int E, int n, int me, int T, int k, int cap,
                           void* const* cnt_ptrs, void* const* flag_ptrs, int parity, unsigned int epoch, void* stream) {
  if (n < 1 || n > MOE_MAX_RANKS || E < 1 || E > MOE_MAX_EXPERTS || (E % n) || me < 0 || me >= n) return LB_ERR_SHAPE;
  PlanParams p;
  p.blk_hist = (const int*)blk_hist; p.blk_psum = (const float*)blk_psum; p.blk_base = (int*)blk_base;
  p.dst_row0 = (int*)dst_row0; p.seg = (int*)seg; p.frac = (float*)frac; p.aux = (float*)aux;
  p.nblk = nblk; p.E = E; p.LE = E / n; p.n = n; p.me = me; p.T = T; p.k = k; p.cap = cap;
  for (int r = 0; r < n; r++) { p.cnt_all[r] = (int*)cnt_ptrs[r]; p.flags[r] = (unsigned int*)flag_ptrs[r]; }
  p.parity = parity & 1; p.epoch = epoch; p.wait_ns = g_lb_flag_wait_ns;
  moe_plan_kernel<<<1, 256, 0, (cudaStream_t)stream>>>(p);
  LB_CHECK_LAUNCH();
  return LB_OK;
}

// dst_ptrs[r] / arrive_ptrs[r]: rank r's destination buffer [cap, H] bf16 and its arrival word.
// compute_rows != 0: rows[t, s] is computed from (within, blk_base, dst_row0) and written;
// otherwise rows is read.  scale [T, k] fp32 or null.  Launches lb_moe_push_ctas(T) CTAs.
extern "C" int lb_moe_push(const void* src, const void* scale, const void* idx, const void* within, const void* blk_base,
                           const void* dst_row0, void* rows, const void* seg, int T, int H, int E, int k, int n, int me,
                           int cap, int compute_rows, void* const* dst_ptrs, void* const* arrive_ptrs, void* stream) {
  if (T <= 0 || (H % 8) || n < 1 || n > MOE_MAX_RANKS || E < 1 || E > MOE_MAX_EXPERTS || (E % n) || k < 1 || k > MOE_MAX_TOPK)
    return LB_ERR_SHAPE;
  PushParams p;
  p.src = (const bf16*)src; p.scale = (const float*)scale; p.idx = (const int*)idx; p.within = (const int*)within;
  p.blk_base = (const int*)blk_base; p.dst_row0 = (const int*)dst_row0; p.rows = (int*)rows; p.seg = (const int*)seg;
  for (int r = 0; r < n; r++) { p.dst[r] = (bf16*)dst_ptrs[r]; p.arrive[r] = (unsigned int*)arrive_ptrs[r]; }
  p.own = p.dst[me];
  p.T = T; p.H = H; p.E = E; p.LE = E / n; p.k = k; p.n = n; p.me = me; p.cap = cap; p.compute_rows = compute_rows;
  moe_push_kernel<<<moe_grid(T), 256, 0, (cudaStream_t)stream>>>(p);
  LB_CHECK_LAUNCH();
  return LB_OK;
}

// src_ptrs[r]: rank r's source buffer [cap, H] bf16; ready_ptrs[r]: rank r's ready words [n] for
// this buffer; epoch grows by one per call on this buffer.  out [T, H] or null; w [T, k] or null;
// dots [T, k] with dots_with [T, H], or both null.
extern "C" int lb_moe_pull(void* out, const void* w, const void* idx, const void* rows, void* dots, const void* dots_with,
                           int T, int H, int E, int k, int n, int me, int cap, void* const* src_ptrs,
                           void* const* ready_ptrs, unsigned int epoch, void* stream) {
  if (T <= 0 || (H % 8) || n < 1 || n > MOE_MAX_RANKS || E < 1 || E > MOE_MAX_EXPERTS || (E % n) || k < 1 || k > MOE_MAX_TOPK)
    return LB_ERR_SHAPE;
  if ((dots == nullptr) != (dots_with == nullptr)) return LB_ERR_ARG;
  PullParams p;
  p.out = (bf16*)out; p.w = (const float*)w; p.idx = (const int*)idx; p.rows = (const int*)rows; p.dots = (float*)dots;
  p.dots_with = (const bf16*)dots_with;
  for (int r = 0; r < n; r++) { p.src[r] = (const bf16*)src_ptrs[r]; p.ready[r] = (unsigned int*)ready_ptrs[r]; }
  p.epoch = epoch; p.wait_ns = g_lb_flag_wait_ns;
  p.T = T; p.H = H; p.E = E; p.LE = E / n; p.k = k; p.n = n; p.me = me; p.cap = cap;
  moe_pull_kernel<<<moe_grid(T), 256, 0, (cudaStream_t)stream>>>(p);
  LB_CHECK_LAUNCH();
  return LB_OK;
}

// dwts [T, k] fp32: gradient of the loss with respect to the routed weights; daux: device pointer to
// the gradient with respect to the load-balance loss (or null); frac [E] from lb_moe_plan.
// dx [T, H] bf16 is written; dwg_acc [E, H] fp32 is added to (zero it first).
extern "C" int lb_moe_router_bwd(const void* x, const void* wg, const void* probs, const void* idx, const void* dwts,
                                 const void* frac, const void* daux, void* dx, void* dwg_acc, int T, int H, int E, int k,
                                 void* stream) {
  if (T <= 0 || (H % 8) || E < 1 || E > MOE_MAX_EXPERTS || k < 1 || k > MOE_MAX_TOPK) return LB_ERR_SHAPE;
  moe_router_bwd_kernel<<<(T + RB_TOKENS - 1) / RB_TOKENS, 256, 0, (cudaStream_t)stream>>>(
      (const bf16*)x, (const bf16*)wg, (const float*)probs, (const int*)idx, (const float*)dwts, (const float*)frac,
      (const float*)daux, (bf16*)dx, (float*)dwg_acc, T, H, E, k);
  LB_CHECK_LAUNCH();
  return LB_OK;
}
