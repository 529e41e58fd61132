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
