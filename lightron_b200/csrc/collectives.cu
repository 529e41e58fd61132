// Stand-alone collectives over NVLink peer memory for small and medium tensors: all-gather,
// reduce-scatter, all-reduce (one-shot peer loads, and an NVLS variant that lets the switch do the
// sum with multimem.ld_reduce / multimem.st) and all-to-all.  One kernel per collective.
//
// Reference counterparts: parallel/communication/all_reduce.py:26-93 (ring reduce-scatter + ring
// all-gather over batch_isend_irecv), ring_all_gather.py:25-58, ring_reduce_scatter.py:25-68 and the
// dist.all_to_all of parallel_cp.py:71.  On an NVSwitch box every peer is one hop away at full
// bandwidth, so instead of N-1 ring steps every rank talks to every peer directly.
//
// Layout.  Every rank owns a staging buffer in peer-visible memory with two halves (calls alternate
// between them: a rank can be at most one call ahead of a peer, because every call waits for every
// peer's flags of that call) and a table of flag words [2][n][G] whose values are call numbers.
// The grid has G CTAs; CTA b of every rank works on slice b of every chunk and only ever waits for
// CTA b of its peers, so no CTA waits for another CTA of its own GPU and the kernels do not depend
// on all G CTAs being resident together.  All waits are bounded (comm.cuh) and report through
// lb_coll_status().
#include "tcgen05.cuh"
#include "comm.cuh"

static __device__ unsigned int g_coll_status[4] = {0, 0, 0, 0};

namespace {

constexpr int COLL_MAX_RANKS = 8;
constexpr int COLL_THREADS = 256;

struct CollParams {
  const void* in;
  void* out;
  uint8_t* stage[COLL_MAX_RANKS];        // rank r's staging buffer (2 halves of half_bytes)
  unsigned int* flags[COLL_MAX_RANKS];   // rank r's flag table [2][n][G]
  uint8_t* mc_stage;                     // NVLS: multicast mapping of the staging buffers (or null)
  long long half_bytes;
  long long chunk_elems;                 // elements per rank-chunk
  int n, me, G, parity;
  unsigned int call;
  unsigned long long wait_ns;
};

__device__ __forceinline__ void coll_fail(unsigned where) {
  if (atomicCAS(&g_coll_status[0], 0u, 1u) == 0u) atomicExch(&g_coll_status[1], where);
}

// this CTA's slice [lo, hi) of a chunk of `elems` elements, in 16-byte vectors of VE elements
__device__ __forceinline__ void slice_of(long long elems, int VE, int G, int b, long long& lo, long long& hi) {
  const long long nvec = (elems + VE - 1) / VE;
  const long long per = (nvec + G - 1) / G;
  lo = min(nvec, per * b) * VE;
  hi = min(elems, min(nvec, per * (b + 1)) * VE);
}

// every thread of the CTA has finished its stores: fence them, then tell CTA b of every rank in `who`
__device__ __forceinline__ void signal_all(const CollParams& p, int kind) {
  __threadfence_system();
  __syncthreads();
  if (threadIdx.x < p.n) {
    __threadfence_system();
    lbcomm::st_release_sys(p.flags[threadIdx.x] + ((size_t)(kind * p.n + p.me) * p.G + blockIdx.x), p.call);
  }
}
__device__ __forceinline__ bool wait_all(const CollParams& p, int kind, int* s_fail) {
  if (threadIdx.x < p.n &&
      !lbcomm::flag_wait_ge(p.flags[p.me] + ((size_t)(kind * p.n + threadIdx.x) * p.G + blockIdx.x), p.call, p.wait_ns)) {
    *s_fail = 1;
    coll_fail(10u + kind);
  }
  __syncthreads();
  return *s_fail == 0;
}

template <typename T> struct Vec;
template <> struct Vec<float> {
  static constexpr int VE = 4;
  static __device__ __forceinline__ void load(const void* p, float* f) { const float4 v = __ldcv(reinterpret_cast<const float4*>(p)); f[0] = v.x; f[1] = v.y; f[2] = v.z; f[3] = v.w; }
  static __device__ __forceinline__ void store(void* p, const float* f) { *reinterpret_cast<float4*>(p) = make_float4(f[0], f[1], f[2], f[3]); }
};
template <> struct Vec<bf16> {
  static constexpr int VE = 8;
  static __device__ __forceinline__ void load(const void* p, float* f) { unpack8(__ldcv(reinterpret_cast<const uint4*>(p)), f); }
  static __device__ __forceinline__ void store(void* p, const float* f) { *reinterpret_cast<uint4*>(p) = pack8(f); }
};

// ---- all-gather: out[s] = in of rank s.  Push, flag, wait, copy out. ------------------------------
template <typename T>
__global__ void __launch_bounds__(COLL_THREADS) all_gather_kernel(const CollParams p) {
  __shared__ int s_fail;
  if (threadIdx.x == 0) s_fail = 0;
  __syncthreads();
  constexpr int VE = Vec<T>::VE;
  long long lo, hi;
  slice_of(p.chunk_elems, VE, p.G, blockIdx.x, lo, hi);
  const T* in = reinterpret_cast<const T*>(p.in);
  const long long half = (long long)p.parity * p.half_bytes;
  for (long long e = lo + (long long)threadIdx.x * VE; e < hi; e += (long long)COLL_THREADS * VE) {
    const uint4 v = *reinterpret_cast<const uint4*>(in + e);
    for (int r = 0; r < p.n; r++)
      *reinterpret_cast<uint4*>(reinterpret_cast<T*>(p.stage[r] + half) + (long long)p.me * p.chunk_elems + e) = v;
  }
  signal_all(p, 0);
  if (!wait_all(p, 0, &s_fail)) return;
  T* out = reinterpret_cast<T*>(p.out);
  const T* mine = reinterpret_cast<const T*>(p.stage[p.me] + half);
  for (int s = 0; s < p.n; s++)
    for (long long e = lo + (long long)threadIdx.x * VE; e < hi; e += (long long)COLL_THREADS * VE)
      *reinterpret_cast<uint4*>(out + (long long)s * p.chunk_elems + e) =
          __ldcv(reinterpret_cast<const uint4*>(mine + (long long)s * p.chunk_elems + e));
}

// ---- all-to-all: out[s] = chunk `me` of rank s's input.  Push chunk j to rank j. ----------------------
template <typename T>
__global__ void __launch_bounds__(COLL_THREADS) all_to_all_kernel(const CollParams p) {
  __shared__ int s_fail;
  if (threadIdx.x == 0) s_fail = 0;
  __syncthreads();
  constexpr int VE = Vec<T>::VE;
  long long lo, hi;
  slice_of(p.chunk_elems, VE, p.G, blockIdx.x, lo, hi);
  const T* in = reinterpret_cast<const T*>(p.in);
  const long long half = (long long)p.parity * p.half_bytes;
  for (int j = 0; j < p.n; j++) {
    const int r = (p.me + j) % p.n;
    for (long long e = lo + (long long)threadIdx.x * VE; e < hi; e += (long long)COLL_THREADS * VE)
      *reinterpret_cast<uint4*>(reinterpret_cast<T*>(p.stage[r] + half) + (long long)p.me * p.chunk_elems + e) =
          *reinterpret_cast<const uint4*>(in + (long long)r * p.chunk_elems + e);
  }
  signal_all(p, 0);
  if (!wait_all(p, 0, &s_fail)) return;
  T* out = reinterpret_cast<T*>(p.out);
  const T* mine = reinterpret_cast<const T*>(p.stage[p.me] + half);
  for (int s = 0; s < p.n; s++)
    for (long long e = lo + (long long)threadIdx.x * VE; e < hi; e += (long long)COLL_THREADS * VE)
      *reinterpret_cast<uint4*>(out + (long long)s * p.chunk_elems + e) =
          __ldcv(reinterpret_cast<const uint4*>(mine + (long long)s * p.chunk_elems + e));
}

// ---- reduce-scatter / all-reduce by peer loads: stage own input, flag, wait, sum over peers ---------
// ALL = false: in holds n chunks, out = sum over ranks of chunk `me`.
// ALL = true : in holds one chunk (the whole tensor), out = sum over ranks of it (one-shot all-reduce).
template <typename T, bool ALL>
__global__ void __launch_bounds__(COLL_THREADS) reduce_kernel(const CollParams p) {
  __shared__ int s_fail;
  if (threadIdx.x == 0) s_fail = 0;
  __syncthreads();
  constexpr int VE = Vec<T>::VE;
  long long lo, hi;
  slice_of(p.chunk_elems, VE, p.G, blockIdx.x, lo, hi);
  const T* in = reinterpret_cast<const T*>(p.in);
  const long long half = (long long)p.parity * p.half_bytes;
  T* mine = reinterpret_cast<T*>(p.stage[p.me] + half);
  const int nchunks = ALL ? 1 : p.n;
  for (int c = 0; c < nchunks; c++)
    for (long long e = lo + (long long)threadIdx.x * VE; e < hi; e += (long long)COLL_THREADS * VE)
      *reinterpret_cast<uint4*>(mine + (long long)c * p.chunk_elems + e) =
          *reinterpret_cast<const uint4*>(in + (long long)c * p.chunk_elems + e);
  signal_all(p, 0);
  if (!wait_all(p, 0, &s_fail)) return;
  T* out = reinterpret_cast<T*>(p.out);
  const long long src_off = ALL ? 0 : (long long)p.me * p.chunk_elems;
  for (long long e = lo + (long long)threadIdx.x * VE; e < hi; e += (long long)COLL_THREADS * VE) {
    float acc[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
    for (int s = 0; s < p.n; s++) {
      float f[8];
      Vec<T>::load(reinterpret_cast<const T*>(p.stage[s] + half) + src_off + e, f);
#pragma unroll
      for (int i = 0; i < VE; i++) acc[i] += f[i];
    }
    Vec<T>::store(out + e, acc);
  }
}

// ---- all-reduce through the switch (NVLS): every rank reduces 1/n of the tensor with one
// multimem.ld_reduce per 16 bytes (the switch reads all n copies and returns the sum) and broadcasts
// the result with multimem.st; two flag rounds frame it. ------------------------------------------------
__device__ __forceinline__ void mm_ld_reduce_f32x4(const void* mc, float* f) {
  asm volatile("multimem.ld_reduce.relaxed.sys.global.add.v4.f32 {%0, %1, %2, %3}, [%4];"
               : "=f"(f[0]), "=f"(f[1]), "=f"(f[2]), "=f"(f[3]) : "l"(mc) : "memory");
}
__device__ __forceinline__ void mm_st_f32x4(void* mc, const float* f) {
  asm volatile("multimem.st.relaxed.sys.global.v4.f32 [%0], {%1, %2, %3, %4};" ::"l"(mc), "f"(f[0]), "f"(f[1]), "f"(f[2]), "f"(f[3]) : "memory");
}
__device__ __forceinline__ void mm_ld_reduce_bf16x8(const void* mc, uint4& v) {
  asm volatile("multimem.ld_reduce.relaxed.sys.global.add.acc::f32.v4.bf16x2 {%0, %1, %2, %3}, [%4];"
               : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(mc) : "memory");
}
__device__ __forceinline__ void mm_st_b32x4(void* mc, const uint4& v) {
  asm volatile("multimem.st.relaxed.sys.global.v4.bf16x2 [%0], {%1, %2, %3, %4};" ::"l"(mc), "r"(v.x), "r"(v.y), "r"(v.z), "r"(v.w) : "memory");
}

template <typename T>
__global__ void __launch_bounds__(COLL_THREADS) all_reduce_nvls_kernel(const CollParams p) {
  __shared__ int s_fail;
  if (threadIdx.x == 0) s_fail = 0;
  __syncthreads();
  constexpr int VE = Vec<T>::VE;
  long long lo, hi;
  slice_of(p.chunk_elems, VE, p.G, blockIdx.x, lo, hi);          // chunk_elems = whole tensor here
  const T* in = reinterpret_cast<const T*>(p.in);
  const long long half = (long long)p.parity * p.half_bytes;
  T* mine = reinterpret_cast<T*>(p.stage[p.me] + half);
  for (long long e = lo + (long long)threadIdx.x * VE; e < hi; e += (long long)COLL_THREADS * VE)
    *reinterpret_cast<uint4*>(mine + e) = *reinterpret_cast<const uint4*>(in + e);
  signal_all(p, 0);
  if (!wait_all(p, 0, &s_fail)) return;
  // this rank reduces vectors me, me + n, me + 2n, ... of the CTA's slice
  T* mc = reinterpret_cast<T*>(p.mc_stage + half);
  const long long nv = (hi - lo + VE - 1) / VE;
  for (long long v = (long long)threadIdx.x * p.n + p.me; v < nv; v += (long long)COLL_THREADS * p.n) {
    const long long e = lo + v * VE;
    if (sizeof(T) == 4) {
      float f[4];
      mm_ld_reduce_f32x4(mc + e, f);
      mm_st_f32x4(mc + e, f);
    } else {
      uint4 r;
      mm_ld_reduce_bf16x8(mc + e, r);
      mm_st_b32x4(mc + e, r);
    }
  }
  signal_all(p, 1);
  if (!wait_all(p, 1, &s_fail)) return;
  T* out = reinterpret_cast<T*>(p.out);
  for (long long e = lo + (long long)threadIdx.x * VE; e < hi; e += (long long)COLL_THREADS * VE)
    *reinterpret_cast<uint4*>(out + e) = __ldcv(reinterpret_cast<const uint4*>(mine + e));
}

// ---- all-gather straight into a peer-visible destination that is reused (parameter gather of the
// sharded engine).  Every rank stores slice b of its shard at offset me * shard into every rank's
// destination, but only after every rank has released the destination's previous contents: the
// `free` words [n] of this rank hold, per peer, how many uses of the destination that peer has
// finished (lb_slot_release).  No staging copy: when the kernel ends the destination is complete. -----
struct GatherParams {
  const bf16* src;                        // this rank's shard [shard_elems]
  bf16* dst[COLL_MAX_RANKS];              // rank r's destination [n * shard_elems]
  unsigned int* arrive[COLL_MAX_RANKS];   // rank r's arrival table [n][G]
  const unsigned int* free_words;         // this rank's table [n]: uses released by peer r
  long long shard_elems;
  int n, me, G;
  unsigned int use;                       // 1, 2, 3, ... per destination
  unsigned long long wait_ns;
};

__global__ void __launch_bounds__(COLL_THREADS) gather_into_kernel(const GatherParams p) {
  __shared__ int s_fail;
  if (threadIdx.x == 0) s_fail = 0;
  __syncthreads();
  if (threadIdx.x < p.n && p.use > 1u && !lbcomm::flag_wait_ge(p.free_words + threadIdx.x, p.use - 1u, p.wait_ns)) {
    s_fail = 1;
    coll_fail(20u);
  }
  __syncthreads();
  if (s_fail) return;
  long long lo, hi;
  slice_of(p.shard_elems, 8, p.G, blockIdx.x, lo, hi);
  for (long long e = lo + (long long)threadIdx.x * 8; e < hi; e += (long long)COLL_THREADS * 8) {
    const uint4 v = *reinterpret_cast<const uint4*>(p.src + e);
    for (int j = 0; j < p.n; j++) {
      const int r = (p.me + 1 + j) % p.n;             // peers first, the local copy last
      *reinterpret_cast<uint4*>(p.dst[r] + (long long)p.me * p.shard_elems + e) = v;
    }
  }
  __threadfence_system();
  __syncthreads();
  if (threadIdx.x < p.n) {
    __threadfence_system();
    lbcomm::st_release_sys(p.arrive[threadIdx.x] + ((size_t)p.me * p.G + blockIdx.x), p.use);
    if (!lbcomm::flag_wait_ge(p.arrive[p.me] + ((size_t)threadIdx.x * p.G + blockIdx.x), p.use, p.wait_ns)) coll_fail(21u);
  }
}

struct ReleaseParams { unsigned int* tab[COLL_MAX_RANKS]; int n, me; unsigned int use; };
__global__ void slot_release_kernel(const ReleaseParams p) {
  if (threadIdx.x < p.n) {
    __threadfence_system();
    lbcomm::st_release_sys(p.tab[threadIdx.x] + p.me, p.use);
  }
}

// ---- context parallelism: gradients of K and V back to the ranks that own the rows -------------------
// After the two attention backward launches of a layer, rank s holds partial dK / dV for the key
// prefixes of its two query chunks: call a covers rows [0, (s+1) n), call b rows [0, (2c-s) n) (zig-zag:
// rank s owns sequence chunks s and 2c-1-s of n rows).  The backward kernels wrote them straight
// into peer-visible buffers; this kernel lets every owner read, for each of its two chunks, the
// partials of the peers whose prefix covers it, sum them in fp32 and store its bf16 dK / dV.
struct CpDkvParams {
  const bf16* ka[COLL_MAX_RANKS];     // rank s's dK of call a: [B, (s+1) n, row_elems]
  const bf16* kb[COLL_MAX_RANKS];     // rank s's dK of call b: [B, (2c-s) n, row_elems]
  const bf16* va[COLL_MAX_RANKS];
  const bf16* vb[COLL_MAX_RANKS];
  unsigned int* ready[COLL_MAX_RANKS];   // rank s's words [c]
  bf16 *out_k, *out_v;                // [B, 2 n, row_elems]: chunk `me`, then chunk 2c-1-me
  int B, n, row_elems, c, me;
  unsigned int epoch;
  unsigned long long wait_ns;
};

__global__ void __launch_bounds__(COLL_THREADS) cp_dkv_reduce_kernel(const CpDkvParams p) {
  __shared__ int s_fail;
  if (threadIdx.x == 0) s_fail = 0;
  __syncthreads();
  if (threadIdx.x < p.c) {
    if (blockIdx.x == 0) {              // this kernel runs behind the launches that wrote this rank's partials
      __threadfence_system();
      lbcomm::st_release_sys(p.ready[threadIdx.x] + p.me, p.epoch);
    }
    if (!lbcomm::flag_wait_ge(p.ready[p.me] + threadIdx.x, p.epoch, p.wait_ns)) { s_fail = 1; coll_fail(30u); }
  }
  __syncthreads();
  if (s_fail) return;
  const int vpr = p.row_elems >> 3;
  const long long total = (long long)p.B * 2 * p.n * vpr;
  for (long long i = (long long)blockIdx.x * COLL_THREADS + threadIdx.x; i < total; i += (long long)gridDim.x * COLL_THREADS) {
    const int v = (int)(i % vpr);
    const long long br = i / vpr;
    const int lr = (int)(br % (2 * p.n));              // local row: [chunk me | chunk 2c-1-me]
    const int b = (int)(br / (2 * p.n));
    const bool second = lr >= p.n;
    const long long grow = second ? (long long)(2 * p.c - 1 - p.me) * p.n + (lr - p.n) : (long long)p.me * p.n + lr;
    float ak[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f}, av[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
    for (int s = 0; s < p.c; s++) {
      float f[8];
      const long long sk_a = (long long)(s + 1) * p.n, sk_b = (long long)(2 * p.c - s) * p.n;
      if (grow < sk_a) {
        const long long o = ((long long)b * sk_a + grow) * p.row_elems + v * 8;
        unpack8(lbcomm::ld_nc_v4(p.ka[s] + o), f);
#pragma unroll
        for (int k = 0; k < 8; k++) ak[k] += f[k];
        unpack8(lbcomm::ld_nc_v4(p.va[s] + o), f);
#pragma unroll
        for (int k = 0; k < 8; k++) av[k] += f[k];
      }
      if (grow < sk_b) {
        const long long o = ((long long)b * sk_b + grow) * p.row_elems + v * 8;
        unpack8(lbcomm::ld_nc_v4(p.kb[s] + o), f);
#pragma unroll
        for (int k = 0; k < 8; k++) ak[k] += f[k];
        unpack8(lbcomm::ld_nc_v4(p.vb[s] + o), f);
#pragma unroll
        for (int k = 0; k < 8; k++) av[k] += f[k];
      }
    }
    const long long oo = ((long long)b * 2 * p.n + lr) * p.row_elems + v * 8;
    *reinterpret_cast<uint4*>(p.out_k + oo) = pack8(ak);
    *reinterpret_cast<uint4*>(p.out_v + oo) = pack8(av);
  }
}

// ---- Ulysses: sequence shards <-> head shards, layout change and RoPE inside the exchange -------------
// mode 0 (before attention): src is the projection output [B * Sl, src_ld] of which columns
//   [col0, col0 + H * d) are H heads; head h of local token (b, sl) is stored into rank h / hl's
//   buffer [B, c * Sl, hl, d] at row me * Sl + sl (hl = H / c heads per rank), rotated on the way when
//   cos / sin are given.  With rep > 1 (fewer KV heads than ranks) head h goes to ranks h * rep ..
//   h * rep + rep - 1, one head per rank.
// mode 1 (after attention): src [B, c * Sl, hl, d]; row (b, s) belongs to rank s / Sl, which receives
//   it at heads me * hl .. me * hl + hl - 1 of a [B * Sl, dst_ld] matrix whose head columns start at
//   dst_col0 (a plain [B, Sl, c * hl, d] tensor, or the q / k / v columns of a fused gradient).
// Both directions are stores into peer-visible destinations (two buffers alternate by call); CTA b of
// a rank signals CTA b of every peer when its stores are fenced and leaves once every peer's CTA b
// has signalled, so at kernel end the whole destination is complete.
struct UlyParams {
  const bf16* src;
  bf16* dst[COLL_MAX_RANKS];
  unsigned int* flags[COLL_MAX_RANKS];     // [n][G]
  const float *cosT, *sinT;                // [positions, d / 2] or null
  const int* pos;                          // global position of local row sl, or null (= me * Sl + sl)
  long long src_ld, col0;                  // mode 0: row stride and first column of the heads in src
  long long dst_ld, dst_col0;              // mode 1: row stride and first column of the heads in dst
  int mode, B, Sl, H, hl, d, rep, inverse;
  int n, me, G;
  unsigned int call;
  unsigned long long wait_ns;
};

__global__ void __launch_bounds__(COLL_THREADS) ulysses_a2a_kernel(const UlyParams p) {
  __shared__ int s_fail;
  if (threadIdx.x == 0) s_fail = 0;
  __syncthreads();
  const int vph = p.d >> 3;                                   // 16-byte vectors per head
  const int S = p.n * p.Sl;
  const long long total = (p.mode == 0 ? (long long)p.B * p.Sl * p.H : (long long)p.B * S * p.hl) * vph;
  const long long per = (total + p.G - 1) / p.G;
  const long long lo = min(total, per * blockIdx.x), hi = min(total, per * (blockIdx.x + 1));
  for (long long i = lo + threadIdx.x; i < hi; i += COLL_THREADS) {
    const int v = (int)(i % vph);
    long long t = i / vph;
    if (p.mode == 0) {
      const int h = (int)(t % p.H); t /= p.H;
      const int sl = (int)(t % p.Sl);
      const int b = (int)(t / p.Sl);
      uint4 raw = *reinterpret_cast<const uint4*>(p.src + ((long long)b * p.Sl + sl) * p.src_ld + p.col0 + (long long)h * p.d + v * 8);
      if (p.cosT) {
        const int ps = p.pos ? p.pos[sl] : p.me * p.Sl + sl;
        float f[8], o[8];
        unpack8(raw, f);
        const float4 c4 = *reinterpret_cast<const float4*>(p.cosT + (size_t)ps * (p.d >> 1) + v * 4);
        float4 s4 = *reinterpret_cast<const float4*>(p.sinT + (size_t)ps * (p.d >> 1) + v * 4);
        if (p.inverse) { s4.x = -s4.x; s4.y = -s4.y; s4.z = -s4.z; s4.w = -s4.w; }
        o[0] = f[0] * c4.x - f[1] * s4.x; o[1] = f[0] * s4.x + f[1] * c4.x;
        o[2] = f[2] * c4.y - f[3] * s4.y; o[3] = f[2] * s4.y + f[3] * c4.y;
        o[4] = f[4] * c4.z - f[5] * s4.z; o[5] = f[4] * s4.z + f[5] * c4.z;
        o[6] = f[6] * c4.w - f[7] * s4.w; o[7] = f[6] * s4.w + f[7] * c4.w;
        raw = pack8(o);
      }
      const long long drow = (long long)b * S + (long long)p.me * p.Sl + sl;
      if (p.rep <= 1) {
        const int r = h / p.hl, hh = h - r * p.hl;
        *reinterpret_cast<uint4*>(p.dst[r] + (drow * p.hl + hh) * p.d + v * 8) = raw;
      } else {
        for (int j = 0; j < p.rep; j++)
          *reinterpret_cast<uint4*>(p.dst[h * p.rep + j] + drow * p.d + v * 8) = raw;
      }
    } else {
      const int h = (int)(t % p.hl); t /= p.hl;
      const int s = (int)(t % S);
      const int b = (int)(t / S);
      const uint4 raw = *reinterpret_cast<const uint4*>(p.src + (((long long)b * S + s) * p.hl + h) * p.d + v * 8);
      const int r = s / p.Sl, sl = s - r * p.Sl;
      *reinterpret_cast<uint4*>(p.dst[r] + ((long long)b * p.Sl + sl) * p.dst_ld + p.dst_col0 + ((long long)p.me * p.hl + h) * p.d + v * 8) = raw;
    }
  }
  __threadfence_system();
  __syncthreads();
  if (threadIdx.x < p.n) {
    __threadfence_system();
    lbcomm::st_release_sys(p.flags[threadIdx.x] + ((size_t)p.me * p.G + blockIdx.x), p.call);
    if (!lbcomm::flag_wait_ge(p.flags[p.me] + ((size_t)threadIdx.x * p.G + blockIdx.x), p.call, p.wait_ns)) coll_fail(40u);
  }
}

// ---- vocab-parallel embedding by peer stores --------------------------------------------------------
// Rank r holds the rows of the table for vocab ids [v0, v1).  The library form (reference
// parallel/parallel_tp.py:131-143) looks up a mostly-zero [T, H] partial on every rank and
// all-reduces (or reduce-scatters) it.  Here every row travels exactly once: the rank that owns a
// token's id stores the row straight into the staging buffer of the rank that needs it (under
// sequence parallelism the owner of row t / rows_per_rank; otherwise every rank), and the receiver
// copies its finished rows out.  CTA b of every rank handles the same slice of the tokens, so CTA b only
// ever waits for CTA b of its peers.  Backward (sequence parallel): every rank publishes its
// gradient rows in its staging buffer and adds, for the tokens whose ids it owns, the rows it reads
// from their owners into its table gradient.
struct EmbParams {
  const long long* tok;                    // [T] token ids (the same on every rank)
  const bf16* w;                           // forward: local table rows [v1 - v0, H]
  bf16* out;                               // forward: [rows kept, H];  backward: table gradient [v1 - v0, H]
  const bf16* dy;                          // backward: this rank's gradient rows [rpr, H]
  bf16* stage[COLL_MAX_RANKS];
  unsigned int* flags[COLL_MAX_RANKS];     // [n][G]
  int T, H, v0, v1, n, me, G, sp, rpr;     // rpr: rows per rank under sp
  unsigned int call;
  unsigned long long wait_ns;
};

__device__ __forceinline__ bool emb_exchange(const EmbParams& p, int* s_fail, unsigned where) {
  __threadfence_system();
  __syncthreads();
  if (threadIdx.x < p.n) {
    __threadfence_system();
    lbcomm::st_release_sys(p.flags[threadIdx.x] + ((size_t)p.me * p.G + blockIdx.x), p.call);
    if (!lbcomm::flag_wait_ge(p.flags[p.me] + ((size_t)threadIdx.x * p.G + blockIdx.x), p.call, p.wait_ns)) {
      *s_fail = 1;
      coll_fail(where);
    }
  }
  __syncthreads();
  return *s_fail == 0;
}

__global__ void __launch_bounds__(COLL_THREADS) embed_tp_fwd_kernel(const EmbParams p) {
  __shared__ int s_fail;
  if (threadIdx.x == 0) s_fail = 0;
  __syncthreads();
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, wpb = COLL_THREADS >> 5;
  const int per = (p.T + p.G - 1) / p.G;
  const int lo = min(p.T, per * (int)blockIdx.x), hi = min(p.T, lo + per);
  const int vpr = p.H >> 3;
  for (int t = lo + warp; t < hi; t += wpb) {
    const long long id = p.tok[t];
    if (id < p.v0 || id >= p.v1) continue;
    const uint4* src = reinterpret_cast<const uint4*>(p.w + (size_t)(id - p.v0) * p.H);
    if (p.sp) {
      const int r = t / p.rpr;
      uint4* dst = reinterpret_cast<uint4*>(p.stage[r] + (size_t)(t - r * p.rpr) * p.H);
      for (int v = lane; v < vpr; v += 32) dst[v] = src[v];
    } else {
      for (int v = lane; v < vpr; v += 32) {
        const uint4 x = src[v];
        for (int j = 0; j < p.n; j++) {
          const int r = (p.me + 1 + j) % p.n;
          reinterpret_cast<uint4*>(p.stage[r] + (size_t)t * p.H)[v] = x;
        }
      }
    }
  }
  if (!emb_exchange(p, &s_fail, 50u)) return;
  const int klo = p.sp ? max(lo, p.me * p.rpr) : lo, khi = p.sp ? min(hi, (p.me + 1) * p.rpr) : hi;
  const int base = p.sp ? p.me * p.rpr : 0;
  for (int t = klo + warp; t < khi; t += wpb) {
    const uint4* src = reinterpret_cast<const uint4*>(p.stage[p.me] + (size_t)(t - base) * p.H);
    uint4* dst = reinterpret_cast<uint4*>(p.out + (size_t)(t - base) * p.H);
    for (int v = lane; v < vpr; v += 32) dst[v] = __ldcg(src + v);
  }
}

__global__ void __launch_bounds__(COLL_THREADS) embed_tp_bwd_kernel(const EmbParams p) {
  __shared__ int s_fail;
  if (threadIdx.x == 0) s_fail = 0;
  __syncthreads();
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, wpb = COLL_THREADS >> 5;
  const int per = (p.T + p.G - 1) / p.G;
  const int lo = min(p.T, per * (int)blockIdx.x), hi = min(p.T, lo + per);
  const int vpr = p.H >> 3;
  const int base = p.me * p.rpr;
  for (int t = max(lo, base) + warp; t < min(hi, base + p.rpr); t += wpb) {
    const uint4* src = reinterpret_cast<const uint4*>(p.dy + (size_t)(t - base) * p.H);
    uint4* dst = reinterpret_cast<uint4*>(p.stage[p.me] + (size_t)(t - base) * p.H);
    for (int v = lane; v < vpr; v += 32) dst[v] = src[v];
  }
  if (!emb_exchange(p, &s_fail, 51u)) return;
  for (int t = lo + warp; t < hi; t += wpb) {
    const long long id = p.tok[t];
    if (id < p.v0 || id >= p.v1) continue;
    const int r = t / p.rpr;
    const bf16* src = p.stage[r] + (size_t)(t - r * p.rpr) * p.H;
    bf162* dst = reinterpret_cast<bf162*>(p.out + (size_t)(id - p.v0) * p.H);
    for (int v = lane; v < vpr; v += 32) {
      const uint4 x = lbcomm::ld_nc_v4(src + v * 8);
      const bf162* h2 = reinterpret_cast<const bf162*>(&x);
#pragma unroll
      for (int i = 0; i < 4; i++) atomicAdd(dst + v * 4 + i, h2[i]);
    }
  }
}

// ---- plain copy into a peer's memory, two ways (the movers of the fused kernels are built on these) ---
// mode 0: every thread loads 16 bytes from local memory and stores them to the destination (UNR loads
//         in flight per thread);
// mode 1: the copy engine of the SM does the work: one thread per CTA issues bulk copies
//         global -> shared (cp.async.bulk, completion on an mbarrier) and shared -> global
//         (cp.async.bulk, bulk groups) of CHUNK bytes through a ring of STAGES buffers; no data passes
//         through registers and every NVLink write is a full CHUNK.
constexpr int PC_CHUNK = 16384, PC_STAGES = 4;

// modes 2 and 3 copy in chunks and publish every chunk the way the movers of the fused kernels do
// (a system-scope fence, then one release-add on a flag word in the destination's memory), so that the
// cost of that protocol can be measured without a GEMM around it:
// mode 2: all threads copy a chunk, fence, CTA barrier, thread 0 adds to the chunk's flag;
// mode 3: warps 0-6 copy and hand finished chunks to warp 7 through shared-memory barriers; warp 7
//         fences and adds to the flag while the others are already copying the next chunk.
__global__ void __launch_bounds__(COLL_THREADS) peer_copy_flag_kernel(const uint4* __restrict__ src, uint4* __restrict__ dst,
                                                                      long long nvec, int mode, long long chunk_vecs,
                                                                      unsigned int* flags) {
  constexpr int UNR = 8;
  const long long nchunks = (nvec + chunk_vecs - 1) / chunk_vecs;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  __shared__ uint64_t full[4];
  __shared__ int done;
  if (threadIdx.x == 0) {
    for (int i = 0; i < 4; i++) bw::mbar_init(bw::smem_u32(&full[i]), 7);
    done = 0;
    bw::mbar_init_fence();
  }
  __syncthreads();
  const int nthr = mode == 2 ? COLL_THREADS : COLL_THREADS - 32;
  int j = 0;
  for (long long c = blockIdx.x; c < nchunks; c += gridDim.x, j++) {
    const long long lo = c * chunk_vecs, hi = min(nvec, lo + chunk_vecs);
    if (mode == 2 || warp < 7) {
      if (mode == 3 && j >= 4) {
        int spins = 0;
        while (*reinterpret_cast<volatile int*>(&done) < j - 3)
          if (++spins > (1 << 26)) { coll_fail(61u); return; }
      }
      long long i = lo + threadIdx.x;
      for (; i + (UNR - 1) * nthr < hi; i += UNR * nthr) {
        uint4 v[UNR];
#pragma unroll
        for (int u = 0; u < UNR; u++) v[u] = src[i + u * nthr];
#pragma unroll
        for (int u = 0; u < UNR; u++) dst[i + u * nthr] = v[u];
      }
      for (; i < hi; i += nthr) dst[i] = src[i];
      if (mode == 2) {
        __threadfence_system();
        __syncthreads();
        if (threadIdx.x == 0) lbcomm::red_release_sys_add(flags + c, 1u);
      } else {
        __syncwarp();
        if (lane == 0) bw::mbar_arrive(bw::smem_u32(&full[j & 3]));
      }
    } else if (lane == 0) {
      bool got = false;
      for (uint32_t spin = 0; spin < (1u << 26) && !got; spin++) got = bw::mbar_try_wait(bw::smem_u32(&full[j & 3]), (uint32_t)(j >> 2) & 1u);
      if (!got) { coll_fail(62u); return; }
      __threadfence_system();
      lbcomm::red_release_sys_add(flags + c, 1u);
      *reinterpret_cast<volatile int*>(&done) = j + 1;
    }
  }
}

__global__ void __launch_bounds__(COLL_THREADS) peer_copy_kernel(const uint4* __restrict__ src, uint4* __restrict__ dst,
                                                                 long long nvec, int mode) {
  if (mode == 0) {
    constexpr int UNR = 8;
    const long long stride = (long long)gridDim.x * COLL_THREADS;
    long long i = (long long)blockIdx.x * COLL_THREADS + threadIdx.x;
    for (; i + (UNR - 1) * stride < nvec; i += UNR * stride) {
      uint4 v[UNR];
#pragma unroll
      for (int u = 0; u < UNR; u++) v[u] = src[i + u * stride];
#pragma unroll
      for (int u = 0; u < UNR; u++) dst[i + u * stride] = v[u];
    }
    for (; i < nvec; i += stride) dst[i] = src[i];
    return;
  }
  extern __shared__ uint8_t pc_smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(pc_smem_raw) + 127) & ~(uintptr_t)127);
  __shared__ uint64_t bars[PC_STAGES];
  if (threadIdx.x == 0) {
    for (int s = 0; s < PC_STAGES; s++) bw::mbar_init(bw::smem_u32(&bars[s]), 1);
    bw::mbar_init_fence();
  }
  __syncthreads();
  if (threadIdx.x != 0) return;
  const long long bytes = nvec * 16;
  const long long nchunks = (bytes + PC_CHUNK - 1) / PC_CHUNK;
  const uint8_t* s8 = reinterpret_cast<const uint8_t*>(src);
  uint8_t* d8 = reinterpret_cast<uint8_t*>(dst);
  // chunk c of this CTA is global chunk blockIdx.x + c * gridDim.x; loads run STAGES - 1 chunks ahead
  const long long mine = (nchunks - blockIdx.x + gridDim.x - 1) / gridDim.x;
  auto chunk_bytes = [&](long long c) {
    const long long off = (blockIdx.x + c * gridDim.x) * (long long)PC_CHUNK;
    return (unsigned)min((long long)PC_CHUNK, bytes - off);
  };
  auto issue_load = [&](long long c) {
    const int st = (int)(c % PC_STAGES);
    const long long off = (blockIdx.x + c * gridDim.x) * (long long)PC_CHUNK;
    const unsigned nb = chunk_bytes(c);
    const uint32_t bar = bw::smem_u32(&bars[st]);
    bw::mbar_expect_tx(bar, nb);
    asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
                 ::"r"(bw::smem_u32(smem + st * PC_CHUNK)), "l"(s8 + off), "r"(nb), "r"(bar) : "memory");
  };
  for (long long c = 0; c < min(mine, (long long)PC_STAGES - 1); c++) issue_load(c);
  for (long long c = 0; c < mine; c++) {
    const int st = (int)(c % PC_STAGES);
    const uint32_t phase = (uint32_t)((c / PC_STAGES) & 1);
    int spins = 0;
    while (!bw::mbar_test_wait(bw::smem_u32(&bars[st]), phase)) {
      if (++spins > (1 << 24)) { coll_fail(60u); return; }
    }
    const long long off = (blockIdx.x + c * gridDim.x) * (long long)PC_CHUNK;
    asm volatile("cp.async.bulk.global.shared::cta.bulk_group [%0], [%1], %2;"
                 ::"l"(d8 + off), "r"(bw::smem_u32(smem + st * PC_CHUNK)), "r"(chunk_bytes(c)) : "memory");
    bw::bulk_commit();
    if (c + PC_STAGES - 1 < mine) {
      // the buffer the next load overwrites was the source of the store issued one iteration ago
      asm volatile("cp.async.bulk.wait_group.read 1;" ::: "memory");
      issue_load(c + PC_STAGES - 1);
    }
  }
  asm volatile("cp.async.bulk.wait_group 0;" ::: "memory");
}

int fill(CollParams& p, const void* in, void* out, void* const* stage_ptrs, void* const* flag_ptrs, long long half_bytes,
         long long chunk_elems, int elem_bytes, long long staged_elems, int n, int me, int G, unsigned int call) {
  if (n < 1 || n > COLL_MAX_RANKS || me < 0 || me >= n || G < 1 || chunk_elems <= 0) return LB_ERR_SHAPE;
  if (elem_bytes != 2 && elem_bytes != 4) return LB_ERR_SHAPE;
  if ((chunk_elems * elem_bytes) % 16) return LB_ERR_SHAPE;                 // chunks start on 16-byte boundaries
  if (staged_elems * elem_bytes > half_bytes) return LB_ERR_CAPACITY;
  if (((uintptr_t)in | (uintptr_t)out) & 15) return LB_ERR_ARG;
  p.in = in; p.out = out;
  for (int r = 0; r < n; r++) { p.stage[r] = (uint8_t*)stage_ptrs[r]; p.flags[r] = (unsigned int*)flag_ptrs[r]; }
  p.mc_stage = nullptr;
  p.half_bytes = half_bytes; p.chunk_elems = chunk_elems; p.n = n; p.me = me; p.G = G; p.parity = (int)(call & 1u);
  p.call = call; p.wait_ns = g_lb_flag_wait_ns;
  return LB_OK;
}

}  // namespace

extern "C" int lb_coll_status(void* out) {
  cudaError_t e = cudaMemcpyFromSymbol(out, g_coll_status, sizeof(unsigned int) * 4);
  if (e != cudaSuccess) { g_lb_last_cuda_error = (int)e; return LB_ERR_LAUNCH; }
  unsigned int zeros[4] = {0, 0, 0, 0};
  cudaMemcpyToSymbol(g_coll_status, zeros, sizeof(zeros));
  return LB_OK;
}

// Common arguments: stage_ptrs[r] / flag_ptrs[r] = rank r's staging buffer (2 * half_bytes) and flag
// table (2 * n * G u32, zeroed once); `call` = 1, 2, 3, ... the same on every rank; G CTAs (the same on
// every rank, and the G the flag table was sized for); elem_bytes 2 (bf16) or 4 (fp32); all byte
// counts multiples of 16.  op: 0 all-gather (in: chunk, out: n chunks), 1 all-to-all (n chunks both),
// 2 reduce-scatter (in: n chunks, out: chunk), 3 all-reduce by peer loads (chunk = whole tensor).
extern "C" int lb_collective(int op, const void* in, void* out, void* const* stage_ptrs, void* const* flag_ptrs,
                             long long half_bytes, long long chunk_elems, int elem_bytes, int n, int me, int G,
                             unsigned int call, void* stream) {
  CollParams p;
  const long long staged = (op == 3) ? chunk_elems : chunk_elems * n;
  int rc = fill(p, in, out, stage_ptrs, flag_ptrs, half_bytes, chunk_elems, elem_bytes, staged, n, me, G, call);
  if (rc) return rc;
  cudaStream_t s = (cudaStream_t)stream;
  const bool f32 = elem_bytes == 4;
  switch (op) {
    case 0: if (f32) all_gather_kernel<float><<<G, COLL_THREADS, 0, s>>>(p); else all_gather_kernel<bf16><<<G, COLL_THREADS, 0, s>>>(p); break;
    case 1: if (f32) all_to_all_kernel<float><<<G, COLL_THREADS, 0, s>>>(p); else all_to_all_kernel<bf16><<<G, COLL_THREADS, 0, s>>>(p); break;
    case 2: if (f32) reduce_kernel<float, false><<<G, COLL_THREADS, 0, s>>>(p); else reduce_kernel<bf16, false><<<G, COLL_THREADS, 0, s>>>(p); break;
    case 3: if (f32) reduce_kernel<float, true><<<G, COLL_THREADS, 0, s>>>(p); else reduce_kernel<bf16, true><<<G, COLL_THREADS, 0, s>>>(p); break;
    default: return LB_ERR_ARG;
  }
  LB_CHECK_LAUNCH();
  return LB_OK;
}

// All-reduce with the sum done inside the NVSwitch.  mc_stage: the multicast address that maps the
// staging buffers of all ranks (torch symmetric memory's multicast_ptr).
extern "C" int lb_all_reduce_nvls(const void* in, void* out, void* const* stage_ptrs, void* mc_stage,
                                  void* const* flag_ptrs, long long half_bytes, long long elems, int elem_bytes, int n,
                                  int me, int G, unsigned int call, void* stream) {
  if (mc_stage == nullptr) return LB_ERR_ARG;
  CollParams p;
  int rc = fill(p, in, out, stage_ptrs, flag_ptrs, half_bytes, elems, elem_bytes, elems, n, me, G, call);
  if (rc) return rc;
  p.mc_stage = (uint8_t*)mc_stage;
  cudaStream_t s = (cudaStream_t)stream;
  if (elem_bytes == 4) all_reduce_nvls_kernel<float><<<G, COLL_THREADS, 0, s>>>(p);
  else all_reduce_nvls_kernel<bf16><<<G, COLL_THREADS, 0, s>>>(p);
  LB_CHECK_LAUNCH();
  return LB_OK;
}

// Parameter gather of the sharded engine: src = this rank's bf16 shard, dst_ptrs[r] = rank r's
// destination [n * shard_elems], arrive_ptrs[r] = rank r's arrival table [n][G] u32, free_words = this
// rank's table [n] of released uses; `use` counts the gathers into this destination (1, 2, ...).
extern "C" int lb_gather_into(const void* src, void* const* dst_ptrs, void* const* arrive_ptrs, const void* free_words,
                              long long shard_elems, int n, int me, int G, unsigned int use, void* stream) {
  if (n < 1 || n > COLL_MAX_RANKS || me < 0 || me >= n || G < 1 || shard_elems <= 0 || (shard_elems % 8) || use == 0)
    return LB_ERR_SHAPE;
  GatherParams p;
  p.src = (const bf16*)src;
  for (int r = 0; r < n; r++) { p.dst[r] = (bf16*)dst_ptrs[r]; p.arrive[r] = (unsigned int*)arrive_ptrs[r]; }
  p.free_words = (const unsigned int*)free_words; p.shard_elems = shard_elems; p.n = n; p.me = me; p.G = G; p.use = use;
  p.wait_ns = g_lb_flag_wait_ns;
  gather_into_kernel<<<G, COLL_THREADS, 0, (cudaStream_t)stream>>>(p);
  LB_CHECK_LAUNCH();
  return LB_OK;
}

// Tells every rank that this rank has finished use number `use` of a gather destination.
extern "C" int lb_slot_release(void* const* free_ptrs, int n, int me, unsigned int use, void* stream) {
  if (n < 1 || n > COLL_MAX_RANKS || me < 0 || me >= n) return LB_ERR_SHAPE;
  ReleaseParams p;
  for (int r = 0; r < n; r++) p.tab[r] = (unsigned int*)free_ptrs[r];
  p.n = n; p.me = me; p.use = use;
  slot_release_kernel<<<1, 32, 0, (cudaStream_t)stream>>>(p);
  LB_CHECK_LAUNCH();
  return LB_OK;
}

// Context-parallel dK / dV: ka / kb / va / vb: host arrays of c pointers (rank s's partials of its
// call a / call b, see cp_dkv_reduce_kernel), ready_ptrs[s]: rank s's ready words [c]; epoch grows by
// one per call on these words.  out_k / out_v: [B, 2 n, row_elems] bf16.
extern "C" int lb_cp_dkv_reduce(void* const* ka, void* const* kb, void* const* va, void* const* vb, void* const* ready_ptrs,
                                void* out_k, void* out_v, int B, int n, int row_elems, int c, int me, unsigned int epoch,
                                void* stream) {
  if (c < 1 || c > COLL_MAX_RANKS || me < 0 || me >= c || B <= 0 || n <= 0 || (row_elems % 8)) return LB_ERR_SHAPE;
  CpDkvParams p;
  for (int s = 0; s < c; s++) {
    p.ka[s] = (const bf16*)ka[s]; p.kb[s] = (const bf16*)kb[s]; p.va[s] = (const bf16*)va[s]; p.vb[s] = (const bf16*)vb[s];
    p.ready[s] = (unsigned int*)ready_ptrs[s];
  }
  p.out_k = (bf16*)out_k; p.out_v = (bf16*)out_v; p.B = B; p.n = n; p.row_elems = row_elems; p.c = c; p.me = me;
  p.epoch = epoch; p.wait_ns = g_lb_flag_wait_ns;
  const long long total = (long long)B * 2 * n * (row_elems / 8);
  long long blocks = (total + COLL_THREADS - 1) / COLL_THREADS;
  const long long cap = (long long)lb_num_sms() * 8;
  if (blocks > cap) blocks = cap;
  cp_dkv_reduce_kernel<<<(int)blocks, COLL_THREADS, 0, (cudaStream_t)stream>>>(p);
  LB_CHECK_LAUNCH();
  return LB_OK;
}

// Ulysses exchange (see ulysses_a2a_kernel).  dst_ptrs[r] / flag_ptrs[r]: rank r's destination buffer
// and flag table [n][G] u32 (zeroed once); call = 1, 2, ... per flag table.  cosT / sinT / pos may be null.
extern "C" int lb_ulysses_a2a(int mode, const void* src, long long src_ld, long long col0, long long dst_ld,
                              long long dst_col0, void* const* dst_ptrs,
                              void* const* flag_ptrs, const void* cosT, const void* sinT, const void* pos, int inverse, int B,
                              int Sl, int H, int hl, int d, int rep, int n, int me, int G, unsigned int call, void* stream) {
  if (n < 1 || n > COLL_MAX_RANKS || me < 0 || me >= n || B <= 0 || Sl <= 0 || (d % 8) || G < 1) return LB_ERR_SHAPE;
  if (mode == 0 && ((src_ld % 8) || (col0 % 8))) return LB_ERR_SHAPE;
  if (mode == 1 && ((dst_ld % 8) || (dst_col0 % 8))) return LB_ERR_SHAPE;
  if (mode == 0 && rep <= 1 && hl * n != H) return LB_ERR_SHAPE;
  if (mode == 0 && rep > 1 && H * rep != n) return LB_ERR_SHAPE;
  if ((cosT == nullptr) != (sinT == nullptr)) return LB_ERR_ARG;
  UlyParams p;
  p.src = (const bf16*)src;
  for (int r = 0; r < n; r++) { p.dst[r] = (bf16*)dst_ptrs[r]; p.flags[r] = (unsigned int*)flag_ptrs[r]; }
  p.cosT = (const float*)cosT; p.sinT = (const float*)sinT; p.pos = (const int*)pos; p.src_ld = src_ld; p.col0 = col0; p.dst_ld = dst_ld; p.dst_col0 = dst_col0;
  p.mode = mode; p.B = B; p.Sl = Sl; p.H = H; p.hl = hl; p.d = d; p.rep = rep; p.inverse = inverse;
  p.n = n; p.me = me; p.G = G; p.call = call; p.wait_ns = g_lb_flag_wait_ns;
  ulysses_a2a_kernel<<<G, COLL_THREADS, 0, (cudaStream_t)stream>>>(p);
  LB_CHECK_LAUNCH();
  return LB_OK;
}

// Vocab-parallel embedding over peer memory (see embed_tp_fwd_kernel).  tok [T] int64, w this rank's
// rows [v1 - v0, H]; stage_ptrs[r] / flag_ptrs[r]: rank r's staging buffer of this call's parity
// ([T / n, H] under sp, else [T, H]) and flag table [n][G] (zeroed once; `call` = 1, 2, ... per table).
// sp != 0: out receives this rank's T / n rows (T a multiple of n); sp == 0: all T rows.
extern "C" int lb_embed_tp_fwd(const void* tok, const void* w, void* out, void* const* stage_ptrs, void* const* flag_ptrs,
                               int T, int H, int v0, int v1, int n, int me, int G, int sp, unsigned int call, void* stream) {
  if (n < 1 || n > COLL_MAX_RANKS || me < 0 || me >= n || G < 1 || T <= 0 || H <= 0 || (H % 8) || (sp && T % n)) return LB_ERR_SHAPE;
  if (((uintptr_t)w | (uintptr_t)out) & 15) return LB_ERR_ARG;
  EmbParams p;
  p.tok = (const long long*)tok; p.w = (const bf16*)w; p.out = (bf16*)out; p.dy = nullptr;
  for (int r = 0; r < n; r++) { p.stage[r] = (bf16*)stage_ptrs[r]; p.flags[r] = (unsigned int*)flag_ptrs[r]; }
  p.T = T; p.H = H; p.v0 = v0; p.v1 = v1; p.n = n; p.me = me; p.G = G; p.sp = sp; p.rpr = sp ? T / n : T;
  p.call = call; p.wait_ns = g_lb_flag_wait_ns;
  embed_tp_fwd_kernel<<<G, COLL_THREADS, 0, (cudaStream_t)stream>>>(p);
  LB_CHECK_LAUNCH();
  return LB_OK;
}

// Gradient of the table under sequence parallelism: dy this rank's [T / n, H] rows, dw [v1 - v0, H]
// (accumulated into with bf16 atomics: zero it, or pass a gradient to add to).  stage_ptrs[r]: rank
// r's [T / n, H] staging buffer of this call's parity.
extern "C" int lb_embed_tp_bwd(const void* tok, const void* dy, void* dw, void* const* stage_ptrs, void* const* flag_ptrs,
                               int T, int H, int v0, int v1, int n, int me, int G, unsigned int call, void* stream) {
  if (n < 1 || n > COLL_MAX_RANKS || me < 0 || me >= n || G < 1 || T <= 0 || H <= 0 || (H % 8) || (T % n)) return LB_ERR_SHAPE;
  if (((uintptr_t)dy | (uintptr_t)dw) & 15) return LB_ERR_ARG;
  EmbParams p;
  p.tok = (const long long*)tok; p.w = nullptr; p.out = (bf16*)dw; p.dy = (const bf16*)dy;
  for (int r = 0; r < n; r++) { p.stage[r] = (bf16*)stage_ptrs[r]; p.flags[r] = (unsigned int*)flag_ptrs[r]; }
  p.T = T; p.H = H; p.v0 = v0; p.v1 = v1; p.n = n; p.me = me; p.G = G; p.sp = 1; p.rpr = T / n;
  p.call = call; p.wait_ns = g_lb_flag_wait_ns;
  embed_tp_bwd_kernel<<<G, COLL_THREADS, 0, (cudaStream_t)stream>>>(p);
  LB_CHECK_LAUNCH();
  return LB_OK;
}

// Copy `bytes` (a multiple of 16) from local memory to dst, which may be a peer's memory, with `ctas`
// CTAs.  mode 0: 16-byte loads and stores by every thread; mode 1: bulk copies through shared memory
// issued by one thread per CTA.  The measured rate of this call is the ceiling of what the movers inside
// the fused kernels can reach.
// modes 2 / 3 (see peer_copy_flag_kernel): `chunk_bytes` per published chunk, `flags`: one zeroed u32
// per chunk in the destination GPU's memory.
extern "C" int lb_peer_copy_flagged(const void* src, void* dst, long long bytes, int mode, int ctas, long long chunk_bytes,
                                    void* flags, void* stream) {
  if (bytes <= 0 || (bytes % 16) || ctas < 1 || mode < 2 || mode > 3 || chunk_bytes < 16 || (chunk_bytes % 16) || !flags) return LB_ERR_SHAPE;
  if (((uintptr_t)src | (uintptr_t)dst) & 15) return LB_ERR_ARG;
  peer_copy_flag_kernel<<<ctas, COLL_THREADS, 0, (cudaStream_t)stream>>>((const uint4*)src, (uint4*)dst, bytes / 16, mode,
                                                                        chunk_bytes / 16, (unsigned int*)flags);
  LB_CHECK_LAUNCH();
  return LB_OK;
}

extern "C" int lb_peer_copy(const void* src, void* dst, long long bytes, int mode, int ctas, void* stream) {
  if (bytes <= 0 || (bytes % 16) || ctas < 1 || mode < 0 || mode > 1) return LB_ERR_SHAPE;
  if (((uintptr_t)src | (uintptr_t)dst) & 15) return LB_ERR_ARG;
  const int smem = mode == 1 ? PC_STAGES * PC_CHUNK + 128 : 0;
  if (mode == 1) {
    static bool attr_set = false;
    if (!attr_set) {
      cudaFuncSetAttribute(peer_copy_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, PC_STAGES * PC_CHUNK + 128);
      attr_set = true;
    }
  }
  peer_copy_kernel<<<ctas, COLL_THREADS, smem, (cudaStream_t)stream>>>((const uint4*)src, (uint4*)dst, bytes / 16, mode);
  LB_CHECK_LAUNCH();
  return LB_OK;
}
