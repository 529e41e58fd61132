// Data-parallel gradient reduce-scatter + AdamW + parameter all-gather in ONE kernel over
// NVLink peer memory.
//
// Every rank of the replica group keeps its bf16 gradient arena and its bf16 parameter arena
// in symmetric memory (mapped by all peers) and owns 1/n of the elements: fp32 master weights and
// Adam moments exist only for that shard.  For its shard a rank
//   1. loads the gradient from every replica with 16-byte peer loads and sums them in fp32
//      (the reduce-scatter, with the bf16 -> fp32 cast and the 1/n scaling folded in),
//   2. applies the decoupled-weight-decay Adam update to master / m / v (local fp32),
//   3. stores the new bf16 parameters into every replica's parameter arena with 16-byte peer
//      stores (the all-gather).
// The same kernel serves the fully sharded engine (parallel/fsdp.py), one launch per block of the
// model as its backward completes: there the reduced gradient can first be accumulated into an fp32
// shard over several micro-batches (`acc`, with `do_update` only on the last), and the new bf16
// parameters go to this rank's shard only (`push_all` = 0): the next forward gathers them.
// The whole GPU takes part (hundreds of thousands of independent 16-byte loads in flight cover
// the NVLink latency).  Two flag exchanges frame the kernel: "my gradients are complete" before any
// peer load, and "my parameter pushes have landed" before the kernel may end, so that the next
// forward on this stream sees every shard.  Waits are bounded and report through lb_dp_status().
#include "comm.cuh"

static __device__ unsigned int g_dp_status[4] = {0, 0, 0, 0};

namespace {

constexpr int MAX_RANKS = 8;

struct DpParams {
  const bf16* grad[MAX_RANKS];     // every replica's gradient arena (peer pointers)
  bf16* param[MAX_RANKS];          // every replica's parameter arena
  unsigned int* flags[MAX_RANKS];  // every replica's flag words: [0..7] ready, [8..15] done
  unsigned int* block_counter;     // local
  float *master, *m, *v;           // local shard state, shard_len elements
  long long shard_start, shard_len;
  int n, rank;
  unsigned int epoch;
  float lr, b1, b2, eps, wd, bc1, bc2, gscale;
  unsigned long long wait_ns;      // limit of the two flag waits
  float* acc;                      // fp32 gradient accumulator of the shard, or null
  int do_update;                   // 0: only add the reduced gradient to acc
  int push_all;                    // 1: new parameters go to every replica's arena, 0: to param[rank] only
};

using lbcomm::st_release_sys;

// A wait that ran out records where and makes the caller skip its share of the update: master
// weights, moments and parameters of that block's range keep their old values, and the host sees
// the status word at its next read (lb_dp_status), before it can checkpoint or go on training.
__device__ __forceinline__ bool wait_ge(const unsigned int* f, unsigned int target, unsigned long long limit_ns, unsigned where) {
  if (lbcomm::flag_wait_ge(f, target, limit_ns)) return true;
  atomicExch(&g_dp_status[0], 1u);
  atomicExch(&g_dp_status[1], where);
  return false;
}

__global__ void __launch_bounds__(256) dp_adamw_kernel(const DpParams p) {
  // ---- first flag exchange: gradients of every replica are complete ----
  if (blockIdx.x == 0 && threadIdx.x < p.n) {
    __threadfence_system();
    st_release_sys(p.flags[threadIdx.x] + p.rank, p.epoch);
  }
  __shared__ int s_failed;
  if (threadIdx.x == 0) s_failed = 0;
  __syncthreads();
  if (threadIdx.x < p.n && !wait_ge(p.flags[p.rank] + threadIdx.x, p.epoch, p.wait_ns, 1u)) s_failed = 1;
  __syncthreads();
  const bool failed = s_failed != 0;       // some replica's gradients never became ready: touch nothing

  const float inv_bc2_sqrt = rsqrtf(p.bc2);
  const float step = p.lr / p.bc1;
  const float gs = p.gscale / (float)p.n;
  const long long nvec = p.shard_len / 8;
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < nvec && !failed; i += (long long)gridDim.x * blockDim.x) {
    const long long e = p.shard_start + i * 8;
    float g[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
    for (int r = 0; r < p.n; r++) {
      float f[8];
      unpack8(__ldcv(reinterpret_cast<const uint4*>(p.grad[r] + e)), f);   // never a stale cached line
#pragma unroll
      for (int k = 0; k < 8; k++) g[k] += f[k];
    }
    if (p.acc) {
      float a[8];
      *reinterpret_cast<float4*>(a) = *reinterpret_cast<const float4*>(p.acc + i * 8);
      *reinterpret_cast<float4*>(a + 4) = *reinterpret_cast<const float4*>(p.acc + i * 8 + 4);
#pragma unroll
      for (int k = 0; k < 8; k++) g[k] += a[k];
      if (!p.do_update) {
        *reinterpret_cast<float4*>(p.acc + i * 8) = *reinterpret_cast<const float4*>(g);
        *reinterpret_cast<float4*>(p.acc + i * 8 + 4) = *reinterpret_cast<const float4*>(g + 4);
        continue;
      }
      *reinterpret_cast<float4*>(p.acc + i * 8) = make_float4(0.f, 0.f, 0.f, 0.f);
      *reinterpret_cast<float4*>(p.acc + i * 8 + 4) = make_float4(0.f, 0.f, 0.f, 0.f);
    }
    float w[8], mm[8], vv[8];
    *reinterpret_cast<float4*>(w) = *reinterpret_cast<const float4*>(p.master + i * 8);
    *reinterpret_cast<float4*>(w + 4) = *reinterpret_cast<const float4*>(p.master + i * 8 + 4);
    *reinterpret_cast<float4*>(mm) = *reinterpret_cast<const float4*>(p.m + i * 8);
    *reinterpret_cast<float4*>(mm + 4) = *reinterpret_cast<const float4*>(p.m + i * 8 + 4);
    *reinterpret_cast<float4*>(vv) = *reinterpret_cast<const float4*>(p.v + i * 8);
    *reinterpret_cast<float4*>(vv + 4) = *reinterpret_cast<const float4*>(p.v + i * 8 + 4);
#pragma unroll
    for (int k = 0; k < 8; k++) {
      const float gg = g[k] * gs;
      float x = w[k] * (1.f - p.lr * p.wd);
      mm[k] = p.b1 * mm[k] + (1.f - p.b1) * gg;
      vv[k] = p.b2 * vv[k] + (1.f - p.b2) * gg * gg;
      x -= step * mm[k] / (sqrtf(vv[k]) * inv_bc2_sqrt + p.eps);
      w[k] = x;
    }
    *reinterpret_cast<float4*>(p.master + i * 8) = *reinterpret_cast<const float4*>(w);
    *reinterpret_cast<float4*>(p.master + i * 8 + 4) = *reinterpret_cast<const float4*>(w + 4);
    *reinterpret_cast<float4*>(p.m + i * 8) = *reinterpret_cast<const float4*>(mm);
    *reinterpret_cast<float4*>(p.m + i * 8 + 4) = *reinterpret_cast<const float4*>(mm + 4);
    *reinterpret_cast<float4*>(p.v + i * 8) = *reinterpret_cast<const float4*>(vv);
    *reinterpret_cast<float4*>(p.v + i * 8 + 4) = *reinterpret_cast<const float4*>(vv + 4);
    const uint4 packed = pack8(w);
    if (p.push_all) {
      for (int r = 0; r < p.n; r++) *reinterpret_cast<uint4*>(p.param[r] + e) = packed;
    } else {
      *reinterpret_cast<uint4*>(p.param[p.rank] + e) = packed;
    }
  }

  // ---- second flag exchange: my pushes have landed everywhere; leave only when everybody's have ----
  __threadfence_system();
  __syncthreads();
  __shared__ unsigned int s_last;
  if (threadIdx.x == 0) s_last = (atomicAdd(p.block_counter, 1u) == gridDim.x * p.epoch - 1u) ? 1u : 0u;
  __syncthreads();
  if (s_last) {
    if (threadIdx.x < p.n) {
      __threadfence_system();
      st_release_sys(p.flags[threadIdx.x] + 8 + p.rank, p.epoch);
      wait_ge(p.flags[p.rank] + 8 + threadIdx.x, p.epoch, p.wait_ns, 2u);
    }
  }
}

}  // namespace

extern "C" int lb_dp_status(void* out) {
  cudaError_t e = cudaMemcpyFromSymbol(out, g_dp_status, sizeof(unsigned int) * 4);
  if (e != cudaSuccess) { g_lb_last_cuda_error = (int)e; return LB_ERR_LAUNCH; }
  unsigned int zeros[4] = {0, 0, 0, 0};
  cudaMemcpyToSymbol(g_dp_status, zeros, sizeof(zeros));
  return LB_OK;
}

// grad_ptrs / param_ptrs / flag_ptrs: host arrays of n pointers (rank order of the replica group).
// flag words (16 x u32 per rank) and block_counter (1 x u32, local) are zeroed once; `epoch` and
// `grid_blocks` must be the same on every call (epoch grows by one per call).  shard_start and
// shard_len are in elements, multiples of 8.
static int dp_adamw_launch(void* const* grad_ptrs, void* const* param_ptrs, void* const* flag_ptrs, void* block_counter,
                           void* master, void* m, void* v, long long shard_start, long long shard_len, int n, int rank,
                           unsigned int epoch, float lr, float b1, float b2, float eps, float wd, float bc1, float bc2,
                           float gscale, int grid_blocks, void* acc, int do_update, int push_all, void* stream) {
  if (!do_update && acc == nullptr) return LB_ERR_ARG;
  if (n < 1 || n > MAX_RANKS || shard_len <= 0 || (shard_len % 8) || (shard_start % 8) || grid_blocks < 1) return LB_ERR_SHAPE;
  DpParams p;
  for (int r = 0; r < n; r++) {
    p.grad[r] = (const bf16*)grad_ptrs[r];
    p.param[r] = (bf16*)param_ptrs[r];
    p.flags[r] = (unsigned int*)flag_ptrs[r];
  }
  p.block_counter = (unsigned int*)block_counter;
  p.master = (float*)master; p.m = (float*)m; p.v = (float*)v;
  p.shard_start = shard_start; p.shard_len = shard_len; p.n = n; p.rank = rank; p.epoch = epoch;
  p.wait_ns = g_lb_flag_wait_ns;
  p.acc = (float*)acc; p.do_update = do_update; p.push_all = push_all;
  p.lr = lr; p.b1 = b1; p.b2 = b2; p.eps = eps; p.wd = wd; p.bc1 = bc1; p.bc2 = bc2; p.gscale = gscale;
  dp_adamw_kernel<<<grid_blocks, 256, 0, (cudaStream_t)stream>>>(p);
  LB_CHECK_LAUNCH();
  return LB_OK;
}

extern "C" int lb_dp_adamw(void* const* grad_ptrs, void* const* param_ptrs, void* const* flag_ptrs, void* block_counter,
                           void* master, void* m, void* v, long long shard_start, long long shard_len, int n, int rank,
                           unsigned int epoch, float lr, float b1, float b2, float eps, float wd, float bc1, float bc2,
                           float gscale, int grid_blocks, void* stream) {
  return dp_adamw_launch(grad_ptrs, param_ptrs, flag_ptrs, block_counter, master, m, v, shard_start, shard_len, n, rank,
                         epoch, lr, b1, b2, eps, wd, bc1, bc2, gscale, grid_blocks, nullptr, 1, 1, stream);
}

// The sharded engine's form: `acc` (fp32 [shard_len], zeroed once) collects the reduced gradient of
// micro-batches launched with do_update = 0; the launch with do_update = 1 adds its own reduced
// gradient, steps AdamW and clears acc.  push_all = 0 stores the new bf16 parameters at
// param_ptrs[rank] + shard_start only (pass a pointer such that this lands in the shard buffer).
extern "C" int lb_fsdp_rs_adamw(void* const* grad_ptrs, void* const* param_ptrs, void* const* flag_ptrs, void* block_counter,
                                void* master, void* m, void* v, void* acc, long long shard_start, long long shard_len, int n,
                                int rank, unsigned int epoch, float lr, float b1, float b2, float eps, float wd, float bc1,
                                float bc2, float gscale, int grid_blocks, int do_update, int push_all, void* stream) {
  return dp_adamw_launch(grad_ptrs, param_ptrs, flag_ptrs, block_counter, master, m, v, shard_start, shard_len, n, rank,
                         epoch, lr, b1, b2, eps, wd, bc1, bc2, gscale, grid_blocks, acc, do_update, push_all, stream);
}
