// Memory-bound kernels: RMSNorm (+residual) fwd/bwd, RoPE, SwiGLU fwd/bwd, embedding fwd/bwd,
// vocab-parallel cross-entropy (stats + grad), AdamW with fp32 master weights, sum of squares.
// All activations are bf16 with fp32 math; every access is a 16-byte vector (8 bf16), so row
// lengths and strides must be multiples of 8 elements.
#include "common.cuh"

#include <mutex>

int g_lb_last_cuda_error = 0;
unsigned long long g_lb_flag_wait_ns = 20ull * 1000ull * 1000ull * 1000ull;

extern "C" int lb_last_error() { return g_lb_last_cuda_error; }

// Wall-time limit (ns) after which a kernel stops waiting for a flag of a peer GPU and reports
// through its status word.  Applies to launches made after the call.
extern "C" int lb_set_flag_wait_ns(unsigned long long ns) {
  if (ns == 0) return LB_ERR_ARG;
  g_lb_flag_wait_ns = ns;
  return LB_OK;
}

int lb_num_sms() {
  static int sms[64] = {0};
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return 148;
  if (sms[dev] == 0) {
    int n = 0;
    if (cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || n <= 0) n = 148;
    sms[dev] = n;
  }
  return sms[dev];
}
extern "C" int lb_sm_count() { return lb_num_sms(); }

// ---------------------------------------------------------------------------------------
// RMSNorm.  One warp per row, two passes over the row (the second hits L1/L2).
//   fwd: h = x (+ res);  rstd = rsqrt(mean(h^2) + eps);  y = h * rstd * w
// ---------------------------------------------------------------------------------------
template <bool HAS_RES>
__global__ void __launch_bounds__(256) rmsnorm_fwd_kernel(const bf16* __restrict__ x, const bf16* __restrict__ res,
                                                          const bf16* __restrict__ w, bf16* __restrict__ h,
                                                          bf16* __restrict__ y, float* __restrict__ rstd_out,
                                                          int rows, int cols, float eps) {
  const int lane = threadIdx.x & 31;
  const int warps_per_block = blockDim.x >> 5;
  const int nvec = cols >> 3;
  for (int row = blockIdx.x * warps_per_block + (threadIdx.x >> 5); row < rows; row += gridDim.x * warps_per_block) {
    const uint4* xr = reinterpret_cast<const uint4*>(x + (size_t)row * cols);
    const uint4* rr = HAS_RES ? reinterpret_cast<const uint4*>(res + (size_t)row * cols) : nullptr;
    uint4* hr = HAS_RES ? reinterpret_cast<uint4*>(h + (size_t)row * cols) : nullptr;
    float ss = 0.f;
    for (int v = lane; v < nvec; v += 32) {
      float f[8];
      unpack8(xr[v], f);
      if (HAS_RES) {
        float g[8];
        unpack8(rr[v], g);
#pragma unroll
        for (int i = 0; i < 8; i++) f[i] += g[i];
        uint4 packed = pack8(f);
        hr[v] = packed;
        unpack8(packed, f);  // the norm sees the rounded residual stream, as a separate add would
      }
#pragma unroll
      for (int i = 0; i < 8; i++) ss += f[i] * f[i];
    }
    ss = warp_sum(ss);
    const float rstd = rsqrtf(ss / (float)cols + eps);
    if (lane == 0) rstd_out[row] = rstd;
    const uint4* src = HAS_RES ? reinterpret_cast<const uint4*>(h + (size_t)row * cols) : xr;
    const uint4* wv = reinterpret_cast<const uint4*>(w);
    uint4* yr = reinterpret_cast<uint4*>(y + (size_t)row * cols);
    if (HAS_RES) __syncwarp();
    for (int v = lane; v < nvec; v += 32) {
      float f[8], g[8];
      unpack8(src[v], f);
      unpack8(wv[v], g);
#pragma unroll
      for (int i = 0; i < 8; i++) f[i] = f[i] * rstd * g[i];
      yr[v] = pack8(f);
    }
  }
}

extern "C" int lb_rmsnorm_fwd(const void* x, const void* res, const void* w, void* h, void* y, void* rstd, int rows,
                              int cols, float eps, void* stream) {
  if (cols % 8 || rows <= 0) return LB_ERR_SHAPE;
  int blocks = (rows + 7) / 8;
  if (blocks > lb_num_sms() * 8) blocks = lb_num_sms() * 8;
  cudaStream_t s = (cudaStream_t)stream;
  if (res)
    rmsnorm_fwd_kernel<true><<<blocks, 256, 0, s>>>((const bf16*)x, (const bf16*)res, (const bf16*)w, (bf16*)h,
                                                    (bf16*)y, (float*)rstd, rows, cols, eps);
  else
    rmsnorm_fwd_kernel<false><<<blocks, 256, 0, s>>>((const bf16*)x, nullptr, (const bf16*)w, nullptr, (bf16*)y,
                                                     (float*)rstd, rows, cols, eps);
  LB_CHECK_LAUNCH();
  return LB_OK;
}

// bwd: g = dy * w; xhat = x * rstd; dx = rstd * (g - xhat * mean(g * xhat)) (+ dres);
//      dw[j] = sum_rows dy * xhat, accumulated per block in shared memory and written to
//      partial[block, cols] (scratch), then reduced over blocks by a second kernel.
__global__ void __launch_bounds__(256) rmsnorm_bwd_kernel(const bf16* __restrict__ dy, const bf16* __restrict__ x,
                                                          const bf16* __restrict__ w, const float* __restrict__ rstd,
                                                          const bf16* __restrict__ dres, bf16* __restrict__ dx,
                                                          float* __restrict__ partial, int rows, int cols) {
  extern __shared__ float s_dw[];
  for (int j = threadIdx.x; j < cols; j += blockDim.x) s_dw[j] = 0.f;
  __syncthreads();
  const int lane = threadIdx.x & 31;
  const int warps_per_block = blockDim.x >> 5;
  const int nvec = cols >> 3;
  const uint4* wv = reinterpret_cast<const uint4*>(w);
  for (int row = blockIdx.x * warps_per_block + (threadIdx.x >> 5); row < rows; row += gridDim.x * warps_per_block) {
    const uint4* dyr = reinterpret_cast<const uint4*>(dy + (size_t)row * cols);
    const uint4* xr = reinterpret_cast<const uint4*>(x + (size_t)row * cols);
    const float r = rstd[row];
    float dot = 0.f;
    for (int v = lane; v < nvec; v += 32) {
      float a[8], b[8], c[8];
      unpack8(dyr[v], a);
      unpack8(xr[v], b);
      unpack8(wv[v], c);
#pragma unroll
      for (int i = 0; i < 8; i++) dot += a[i] * c[i] * b[i] * r;
    }
    dot = warp_sum(dot) / (float)cols;
    const uint4* dr = dres ? reinterpret_cast<const uint4*>(dres + (size_t)row * cols) : nullptr;
    uint4* dxr = reinterpret_cast<uint4*>(dx + (size_t)row * cols);
    for (int v = lane; v < nvec; v += 32) {
      float a[8], b[8], c[8], o[8];
      unpack8(dyr[v], a);
      unpack8(xr[v], b);
      unpack8(wv[v], c);
#pragma unroll
      for (int i = 0; i < 8; i++) {
        const float xhat = b[i] * r;
        o[i] = r * (a[i] * c[i] - xhat * dot);
        atomicAdd(&s_dw[i * nvec + v], a[i] * xhat);  // [i][v] layout: lanes hit consecutive banks
      }
      if (dr) {
        float e[8];
        unpack8(dr[v], e);
#pragma unroll
        for (int i = 0; i < 8; i++) o[i] += e[i];
      }
      dxr[v] = pack8(o);
    }
  }
  __syncthreads();
  for (int j = threadIdx.x; j < cols; j += blockDim.x)
    partial[(size_t)blockIdx.x * cols + j] = s_dw[(j & 7) * nvec + (j >> 3)];
}

// Block-per-row version (no shared-memory atomics): the block's T threads cover one row with VPT
// uint4 each (cols = 8 * T * VPT), so a thread owns the same 8*VPT columns of every row and keeps
// their dw partial sums in registers.  RB rows are in flight per iteration; their dy / x stay in
// registers between the dot product (one block reduction per iteration, double-buffered so a single
// barrier suffices) and the dx pass.
template <int VPT, int RB>
__global__ void __launch_bounds__(256, (VPT == 1 ? 3 : (VPT <= 3 ? 2 : 1))) rmsnorm_bwd_blk_kernel(const bf16* __restrict__ dy, const bf16* __restrict__ x,
                                                              const bf16* __restrict__ w, const float* __restrict__ rstd,
                                                              const bf16* __restrict__ dres, bf16* __restrict__ dx,
                                                              float* __restrict__ partial, int rows, int cols) {
  __shared__ float s_red[2][RB][8];
  const int T = blockDim.x, t = threadIdx.x, lane = t & 31, warp = t >> 5, nw = T >> 5;
  const float inv_cols = 1.f / (float)cols;
  float wf[VPT][8], acc[VPT][8];
#pragma unroll
  for (int k = 0; k < VPT; k++) {
    unpack8(reinterpret_cast<const uint4*>(w)[t + T * k], wf[k]);
#pragma unroll
    for (int i = 0; i < 8; i++) acc[k][i] = 0.f;
  }
  int par = 0;
  for (int row0 = blockIdx.x * RB; row0 < rows; row0 += gridDim.x * RB, par ^= 1) {
    uint4 kd[RB][VPT], kx[RB][VPT];
    float r[RB], dot[RB];
#pragma unroll
    for (int rb = 0; rb < RB; rb++) {
      const int row = row0 + rb;
      const bool ok = row < rows;
      r[rb] = ok ? rstd[row] : 0.f;
#pragma unroll
      for (int k = 0; k < VPT; k++) {
        kd[rb][k] = ok ? reinterpret_cast<const uint4*>(dy + (size_t)row * cols)[t + T * k] : make_uint4(0, 0, 0, 0);
        kx[rb][k] = ok ? reinterpret_cast<const uint4*>(x + (size_t)row * cols)[t + T * k] : make_uint4(0, 0, 0, 0);
      }
    }
#pragma unroll
    for (int rb = 0; rb < RB; rb++) {
      float d = 0.f;
#pragma unroll
      for (int k = 0; k < VPT; k++) {
        float a[8], b[8];
        unpack8(kd[rb][k], a);
        unpack8(kx[rb][k], b);
#pragma unroll
        for (int i = 0; i < 8; i++) d += a[i] * wf[k][i] * b[i];
      }
      d = warp_sum(d * r[rb]);
      if (lane == 0) s_red[par][rb][warp] = d;
    }
    __syncthreads();
#pragma unroll
    for (int rb = 0; rb < RB; rb++) {
      float d = 0.f;
      for (int ww = 0; ww < nw; ww++) d += s_red[par][rb][ww];
      dot[rb] = d * inv_cols;
    }
#pragma unroll
    for (int rb = 0; rb < RB; rb++) {
      const int row = row0 + rb;
      if (row >= rows) break;
#pragma unroll
      for (int k = 0; k < VPT; k++) {
        float a[8], b[8], o[8];
        unpack8(kd[rb][k], a);
        unpack8(kx[rb][k], b);
#pragma unroll
        for (int i = 0; i < 8; i++) {
          const float xhat = b[i] * r[rb];
          o[i] = r[rb] * (a[i] * wf[k][i] - xhat * dot[rb]);
          acc[k][i] += a[i] * xhat;
        }
        if (dres) {
          float e[8];
          unpack8(reinterpret_cast<const uint4*>(dres + (size_t)row * cols)[t + T * k], e);
#pragma unroll
          for (int i = 0; i < 8; i++) o[i] += e[i];
        }
        reinterpret_cast<uint4*>(dx + (size_t)row * cols)[t + T * k] = pack8(o);
      }
    }
  }
#pragma unroll
  for (int k = 0; k < VPT; k++) {
    float* dst = partial + (size_t)blockIdx.x * cols + (size_t)(t + T * k) * 8;
    *reinterpret_cast<float4*>(dst) = make_float4(acc[k][0], acc[k][1], acc[k][2], acc[k][3]);
    *reinterpret_cast<float4*>(dst + 4) = make_float4(acc[k][4], acc[k][5], acc[k][6], acc[k][7]);
  }
}

// Launches the block-per-row version when the width fits it (cols = 8 * T * VPT with T a multiple
// of 32, T <= 256, VPT <= 4); returns false otherwise.
static bool rmsnorm_bwd_blk_dispatch(const void* dy, const void* x, const void* w, const void* rstd, const void* dres,
                                     void* dx, void* partial, int rows, int cols, int nblk, cudaStream_t s) {
  const int nvec = cols / 8;
  const int vpt = (nvec + 255) / 256;
  if (vpt > 4 || nvec % vpt) return false;
  const int T = nvec / vpt;
  if (T % 32) return false;
#define LB_RMS_BLK(V, R)                                                                                          \
  rmsnorm_bwd_blk_kernel<V, R><<<nblk, T, 0, s>>>((const bf16*)dy, (const bf16*)x, (const bf16*)w, (const float*)rstd, \
                                                  (const bf16*)dres, (bf16*)dx, (float*)partial, rows, cols)
  switch (vpt) {
    case 1: LB_RMS_BLK(1, 2); break;
    case 2: LB_RMS_BLK(2, 2); break;
    case 3: LB_RMS_BLK(3, 1); break;
    default: LB_RMS_BLK(4, 1); break;
  }
#undef LB_RMS_BLK
  return true;
}

// dw[j] = sum over blocks of partial[b, j]: 32 columns x 32 row lanes per block.
__global__ void __launch_bounds__(1024) rmsnorm_dw_reduce_kernel(const float* __restrict__ partial, bf16* __restrict__ dw,
                                                                 int nblk, int cols) {
  __shared__ float s[32][33];
  const int j = blockIdx.x * 32 + threadIdx.x;
  float v = 0.f;
  if (j < cols)
    for (int b = threadIdx.y; b < nblk; b += 32) v += partial[(size_t)b * cols + j];
  s[threadIdx.y][threadIdx.x] = v;
  __syncthreads();
  if (threadIdx.y == 0 && j < cols) {
    float t = 0.f;
#pragma unroll
    for (int k = 0; k < 32; k++) t += s[k][threadIdx.x];
    dw[j] = __float2bfloat16(t);
  }
}

// Number of blocks (= rows of the `partial` scratch) that lb_rmsnorm_bwd uses for this shape.
extern "C" int lb_rmsnorm_bwd_blocks(int rows, int cols) {
  // as many blocks as are resident at once (one wave of the grid-stride loop): the block-per-row
  // kernel fits 3 / 2 / 2 / 1 blocks per SM for 1 / 2 / 3 / 4 vectors per thread, the atomics
  // version 2
  const int nvec = cols / 8;
  const int vpt = (nvec + 255) / 256;
  const bool blk = vpt <= 4 && nvec % vpt == 0 && (nvec / vpt) % 32 == 0;
  const int per_sm = !blk ? 2 : (vpt == 1 ? 3 : (vpt <= 3 ? 2 : 1));
  int blocks = (rows + 7) / 8;
  if (blocks > lb_num_sms() * per_sm) blocks = lb_num_sms() * per_sm;
  return blocks < 1 ? 1 : blocks;
}

extern "C" int lb_rmsnorm_bwd(const void* dy, const void* x, const void* w, const void* rstd, const void* dres,
                              void* dx, void* partial, void* dw, int rows, int cols, int nblk, void* stream) {
  if (cols % 8 || rows <= 0 || cols * 4 > 200 * 1024) return LB_ERR_SHAPE;
  if (nblk != lb_rmsnorm_bwd_blocks(rows, cols)) return LB_ERR_ARG;
  cudaStream_t s = (cudaStream_t)stream;
  size_t smem = (size_t)cols * sizeof(float);
  if (rmsnorm_bwd_blk_dispatch(dy, x, w, rstd, dres, dx, partial, rows, cols, nblk, s)) {
    LB_CHECK_LAUNCH();
  } else {
    if (smem > 48 * 1024) cudaFuncSetAttribute(rmsnorm_bwd_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    rmsnorm_bwd_kernel<<<nblk, 256, smem, s>>>((const bf16*)dy, (const bf16*)x, (const bf16*)w, (const float*)rstd,
                                               (const bf16*)dres, (bf16*)dx, (float*)partial, rows, cols);
    LB_CHECK_LAUNCH();
  }
  rmsnorm_dw_reduce_kernel<<<(cols + 31) / 32, dim3(32, 32), 0, s>>>((const float*)partial, (bf16*)dw, nblk, cols);
  LB_CHECK_LAUNCH();
  return LB_OK;
}

// ---------------------------------------------------------------------------------------
// RoPE in place on rows of `t` (row stride ld): the first n_heads*head_dim columns are heads;
// pairs (2i, 2i+1) of every head are rotated by angle pos * theta^(-2i/d).  cos/sin: [*, d/2].
// ---------------------------------------------------------------------------------------
__global__ void rope_kernel(bf16* __restrict__ t, const float* __restrict__ cosT, const float* __restrict__ sinT,
                            const int* __restrict__ positions, int tokens, int S, int n_heads, int head_dim,
                            long long ld, int inverse) {
  const int vec_per_head = head_dim >> 3;
  const long long total = (long long)tokens * n_heads * vec_per_head;
  for (long long idx = (long long)blockIdx.x * blockDim.x + threadIdx.x; idx < total;
       idx += (long long)gridDim.x * blockDim.x) {
    const int v = (int)(idx % vec_per_head);
    const long long th = idx / vec_per_head;
    const int head = (int)(th % n_heads);
    const long long tok = th / n_heads;
    const int s = (int)(tok % S);
    const int pos = positions ? positions[s] : s;
    uint4* p = reinterpret_cast<uint4*>(t + tok * ld + (long long)head * head_dim + v * 8);
    float f[8], o[8];
    unpack8(*p, f);
    const float4 c = *reinterpret_cast<const float4*>(cosT + (size_t)pos * (head_dim >> 1) + v * 4);
    float4 sn = *reinterpret_cast<const float4*>(sinT + (size_t)pos * (head_dim >> 1) + v * 4);
    if (inverse) { sn.x = -sn.x; sn.y = -sn.y; sn.z = -sn.z; sn.w = -sn.w; }
    o[0] = f[0] * c.x - f[1] * sn.x; o[1] = f[0] * sn.x + f[1] * c.x;
    o[2] = f[2] * c.y - f[3] * sn.y; o[3] = f[2] * sn.y + f[3] * c.y;
    o[4] = f[4] * c.z - f[5] * sn.z; o[5] = f[4] * sn.z + f[5] * c.z;
    o[6] = f[6] * c.w - f[7] * sn.w; o[7] = f[6] * sn.w + f[7] * c.w;
    *p = pack8(o);
  }
}

extern "C" int lb_rope(void* t, const void* cosT, const void* sinT, const void* positions, int tokens, int S,
                       int n_heads, int head_dim, long long ld, int inverse, void* stream) {
  if (head_dim % 8 || ld % 8 || tokens <= 0) return LB_ERR_SHAPE;
  long long total = (long long)tokens * n_heads * (head_dim / 8);
  int blocks = (int)((total + 255) / 256);
  if (blocks > lb_num_sms() * 16) blocks = lb_num_sms() * 16;
  rope_kernel<<<blocks, 256, 0, (cudaStream_t)stream>>>((bf16*)t, (const float*)cosT, (const float*)sinT,
                                                        (const int*)positions, tokens, S, n_heads, head_dim, ld,
                                                        inverse);
  LB_CHECK_LAUNCH();
  return LB_OK;
}

// ---------------------------------------------------------------------------------------
// SwiGLU on a fused [rows, 2I] gate|up matrix (row stride ld).
// ---------------------------------------------------------------------------------------
__global__ void swiglu_fwd_kernel(const bf16* __restrict__ gu, bf16* __restrict__ out, int rows, int I, long long ld,
                                  const int* __restrict__ rows_dev) {
  if (rows_dev) rows = max(0, min(rows, *rows_dev));     // row count known only on the device (MoE segments)
  const int vec = I >> 3;
  const long long total = (long long)rows * vec;
  for (long long idx = (long long)blockIdx.x * blockDim.x + threadIdx.x; idx < total;
       idx += (long long)gridDim.x * blockDim.x) {
    const long long r = idx / vec;
    const int v = (int)(idx % vec);
    float g[8], u[8], o[8];
    unpack8(*reinterpret_cast<const uint4*>(gu + r * ld + v * 8), g);
    unpack8(*reinterpret_cast<const uint4*>(gu + r * ld + I + v * 8), u);
#pragma unroll
    for (int i = 0; i < 8; i++) o[i] = g[i] / (1.f + __expf(-g[i])) * u[i];
    *reinterpret_cast<uint4*>(out + r * I + v * 8) = pack8(o);
  }
}

__global__ void swiglu_bwd_kernel(const bf16* __restrict__ gu, const bf16* __restrict__ dy, bf16* __restrict__ dgu,
                                  int rows, int I, long long ld, const int* __restrict__ rows_dev) {
  if (rows_dev) rows = max(0, min(rows, *rows_dev));
  const int vec = I >> 3;
  const long long total = (long long)rows * vec;
  for (long long idx = (long long)blockIdx.x * blockDim.x + threadIdx.x; idx < total;
       idx += (long long)gridDim.x * blockDim.x) {
    const long long r = idx / vec;
    const int v = (int)(idx % vec);
    float g[8], u[8], d[8], dg[8], du[8];
    unpack8(*reinterpret_cast<const uint4*>(gu + r * ld + v * 8), g);
    unpack8(*reinterpret_cast<const uint4*>(gu + r * ld + I + v * 8), u);
    unpack8(*reinterpret_cast<const uint4*>(dy + r * I + v * 8), d);
#pragma unroll
    for (int i = 0; i < 8; i++) {
      const float sig = 1.f / (1.f + __expf(-g[i]));
      dg[i] = d[i] * u[i] * sig * (1.f + g[i] * (1.f - sig));
      du[i] = d[i] * g[i] * sig;
    }
    *reinterpret_cast<uint4*>(dgu + r * 2 * I + v * 8) = pack8(dg);
    *reinterpret_cast<uint4*>(dgu + r * 2 * I + I + v * 8) = pack8(du);
  }
}

static inline int ew_blocks(long long total) {
  long long b = (total + 255) / 256;
  if (b > lb_num_sms() * 16) b = lb_num_sms() * 16;
  return (int)(b < 1 ? 1 : b);
}

// rows_dev (or null): device int; only the first min(rows, *rows_dev) rows are processed.
extern "C" int lb_swiglu_fwd_dev(const void* gu, void* out, int rows, int I, long long ld, const void* rows_dev, void* stream) {
  if (I % 8 || ld % 8 || rows <= 0) return LB_ERR_SHAPE;
  swiglu_fwd_kernel<<<ew_blocks((long long)rows * (I / 8)), 256, 0, (cudaStream_t)stream>>>((const bf16*)gu, (bf16*)out,
                                                                                            rows, I, ld, (const int*)rows_dev);
  LB_CHECK_LAUNCH();
  return LB_OK;
}
extern "C" int lb_swiglu_fwd(const void* gu, void* out, int rows, int I, long long ld, void* stream) {
  return lb_swiglu_fwd_dev(gu, out, rows, I, ld, nullptr, stream);
}

extern "C" int lb_swiglu_bwd_dev(const void* gu, const void* dy, void* dgu, int rows, int I, long long ld,
                                 const void* rows_dev, void* stream) {
  if (I % 8 || ld % 8 || rows <= 0) return LB_ERR_SHAPE;
  swiglu_bwd_kernel<<<ew_blocks((long long)rows * (I / 8)), 256, 0, (cudaStream_t)stream>>>(
      (const bf16*)gu, (const bf16*)dy, (bf16*)dgu, rows, I, ld, (const int*)rows_dev);
  LB_CHECK_LAUNCH();
  return LB_OK;
}
extern "C" int lb_swiglu_bwd(const void* gu, const void* dy, void* dgu, int rows, int I, long long ld, void* stream) {
  return lb_swiglu_bwd_dev(gu, dy, dgu, rows, I, ld, nullptr, stream);
}

// ---------------------------------------------------------------------------------------
// Embedding.  The weight holds vocab ids [v0, v1); ids outside give zero rows (vocab-parallel
// partial result).  Backward scatters with bf16x2 atomics into a zero-initialised dW.
// ---------------------------------------------------------------------------------------
__global__ void embedding_fwd_kernel(const long long* __restrict__ tok, const bf16* __restrict__ w,
                                     bf16* __restrict__ out, int T, int H, int v0, int v1) {
  const int lane = threadIdx.x & 31;
  const int wpb = blockDim.x >> 5;
  const int nvec = H >> 3;
  for (int t = blockIdx.x * wpb + (threadIdx.x >> 5); t < T; t += gridDim.x * wpb) {
    const long long id = tok[t];
    uint4* o = reinterpret_cast<uint4*>(out + (size_t)t * H);
    if (id >= v0 && id < v1) {
      const uint4* src = reinterpret_cast<const uint4*>(w + (size_t)(id - v0) * H);
      for (int v = lane; v < nvec; v += 32) o[v] = src[v];
    } else {
      for (int v = lane; v < nvec; v += 32) o[v] = make_uint4(0, 0, 0, 0);
    }
  }
}

__global__ void embedding_bwd_kernel(const long long* __restrict__ tok, const bf16* __restrict__ dy,
                                     bf16* __restrict__ dw, int T, int H, int v0, int v1) {
  const int lane = threadIdx.x & 31;
  const int wpb = blockDim.x >> 5;
  const int npair = H >> 1;
  for (int t = blockIdx.x * wpb + (threadIdx.x >> 5); t < T; t += gridDim.x * wpb) {
    const long long id = tok[t];
    if (id < v0 || id >= v1) continue;
    const bf162* src = reinterpret_cast<const bf162*>(dy + (size_t)t * H);
    bf162* dst = reinterpret_cast<bf162*>(dw + (size_t)(id - v0) * H);
    for (int v = lane; v < npair; v += 32) atomicAdd(dst + v, src[v]);
  }
}

extern "C" int lb_embedding_fwd(const void* tok, const void* w, void* out, int T, int H, int v0, int v1, void* stream) {
  if (H % 8 || T <= 0) return LB_ERR_SHAPE;
  int blocks = (T + 7) / 8;
  if (blocks > lb_num_sms() * 8) blocks = lb_num_sms() * 8;
  embedding_fwd_kernel<<<blocks, 256, 0, (cudaStream_t)stream>>>((const long long*)tok, (const bf16*)w, (bf16*)out, T,
                                                                 H, v0, v1);
  LB_CHECK_LAUNCH();
  return LB_OK;
}

extern "C" int lb_embedding_bwd(const void* tok, const void* dy, void* dw, int T, int H, int v0, int v1, void* stream) {
  if (H % 8 || T <= 0) return LB_ERR_SHAPE;
  int blocks = (T + 7) / 8;
  if (blocks > lb_num_sms() * 8) blocks = lb_num_sms() * 8;
  embedding_bwd_kernel<<<blocks, 256, 0, (cudaStream_t)stream>>>((const long long*)tok, (const bf16*)dy, (bf16*)dw, T,
                                                                 H, v0, v1);
  LB_CHECK_LAUNCH();
  return LB_OK;
}

// ---------------------------------------------------------------------------------------
// Cross-entropy over [T, V] bf16 logits (row stride ld).  One block per row.
//   stats: row max, sum exp(x - max), and the target's logit if it falls in [v0, v0+V) else 0.
//   grad:  dlogits = (exp(x - lse) - onehot) * (*dloss) * inv_n, written in place if wanted.
// ---------------------------------------------------------------------------------------
__global__ void __launch_bounds__(256) ce_stats_kernel(const bf16* __restrict__ logits, const long long* __restrict__ tgt,
                                                       float* __restrict__ mx_out, float* __restrict__ se_out,
                                                       float* __restrict__ tl_out, int V, long long ld, int v0) {
  const int row = blockIdx.x;
  const uint4* p = reinterpret_cast<const uint4*>(logits + (size_t)row * ld);
  const int nvec = V >> 3;
  float m = -INFINITY, s = 0.f;
  for (int v = threadIdx.x; v < nvec; v += blockDim.x) {
    float f[8];
    unpack8(p[v], f);
    float lm = f[0];
#pragma unroll
    for (int i = 1; i < 8; i++) lm = fmaxf(lm, f[i]);
    const float nm = fmaxf(m, lm);
    float acc = 0.f;
#pragma unroll
    for (int i = 0; i < 8; i++) acc += __expf(f[i] - nm);
    s = s * __expf(m - nm) + acc;
    m = nm;
  }
  __shared__ float sm[8], ss[8];
  const int lane = threadIdx.x & 31, wid = threadIdx.x >> 5;
  float wm = warp_max(m);
  s = warp_sum(m == -INFINITY ? 0.f : s * __expf(m - wm));   // lanes without elements (V < 8 * threads)
  if (lane == 0) { sm[wid] = wm; ss[wid] = s; }
  __syncthreads();
  if (threadIdx.x == 0) {
    float gm = sm[0];
    const int nw = blockDim.x >> 5;
    for (int i = 1; i < nw; i++) gm = fmaxf(gm, sm[i]);
    float gs = 0.f;
    for (int i = 0; i < nw; i++) gs += (sm[i] == -INFINITY) ? 0.f : ss[i] * __expf(sm[i] - gm);
    mx_out[row] = gm;
    se_out[row] = gs;
    const long long t = tgt[row] - v0;
    tl_out[row] = (t >= 0 && t < V) ? __bfloat162float(logits[(size_t)row * ld + t]) : 0.f;
  }
}

__global__ void __launch_bounds__(256) ce_grad_kernel(const bf16* __restrict__ logits, const long long* __restrict__ tgt,
                                                      const float* __restrict__ lse, bf16* __restrict__ dlogits,
                                                      const float* __restrict__ dloss, int V, long long ld, int v0,
                                                      float inv_n, int ignore_index) {
  const int row = blockIdx.x;
  const long long tg = tgt[row];
  const float scale = (tg == ignore_index) ? 0.f : dloss[0] * inv_n;
  const long long t = tg - v0;
  const float l = lse[row];
  const uint4* p = reinterpret_cast<const uint4*>(logits + (size_t)row * ld);
  uint4* q = reinterpret_cast<uint4*>(dlogits + (size_t)row * ld);
  const int nvec = V >> 3;
  for (int v = threadIdx.x; v < nvec; v += blockDim.x) {
    float f[8];
    unpack8(p[v], f);
#pragma unroll
    for (int i = 0; i < 8; i++) {
      float g = __expf(f[i] - l);
      if ((long long)(v * 8 + i) == t) g -= 1.f;
      f[i] = g * scale;
    }
    q[v] = pack8(f);
  }
}

extern "C" int lb_ce_stats(const void* logits, const void* tgt, void* mx, void* se, void* tl, int T, int V,
                           long long ld, int v0, void* stream) {
  if (V % 8 || ld % 8 || T <= 0) return LB_ERR_SHAPE;
  ce_stats_kernel<<<T, 256, 0, (cudaStream_t)stream>>>((const bf16*)logits, (const long long*)tgt, (float*)mx,
                                                       (float*)se, (float*)tl, V, ld, v0);
  LB_CHECK_LAUNCH();
  return LB_OK;
}

extern "C" int lb_ce_grad(const void* logits, const void* tgt, const void* lse, void* dlogits, const void* dloss, int T,
                          int V, long long ld, int v0, float inv_n, int ignore_index, void* stream) {
  if (V % 8 || ld % 8 || T <= 0) return LB_ERR_SHAPE;
  ce_grad_kernel<<<T, 256, 0, (cudaStream_t)stream>>>((const bf16*)logits, (const long long*)tgt, (const float*)lse,
                                                      (bf16*)dlogits, (const float*)dloss, V, ld, v0, inv_n,
                                                      ignore_index);
  LB_CHECK_LAUNCH();
  return LB_OK;
}

// ---------------------------------------------------------------------------------------
// AdamW (decoupled weight decay, torch.optim.AdamW semantics) on fp32 master weights with bf16
// (or fp32) gradients; writes the updated master and its bf16 copy.  n must be a multiple of 4.
// ---------------------------------------------------------------------------------------
template <typename G>
__global__ void adamw_kernel(float* __restrict__ master, float* __restrict__ m, float* __restrict__ v,
                             const G* __restrict__ grad, bf16* __restrict__ param, long long n, float lr, float b1,
                             float b2, float eps, float wd, float bc1, float bc2, float gscale) {
  const float inv_bc2_sqrt = rsqrtf(bc2);
  const float step = lr / bc1;
  for (long long i = ((long long)blockIdx.x * blockDim.x + threadIdx.x) * 4; i < n;
       i += (long long)gridDim.x * blockDim.x * 4) {
    float4 p = *reinterpret_cast<float4*>(master + i);
    float4 mm = *reinterpret_cast<float4*>(m + i);
    float4 vv = *reinterpret_cast<float4*>(v + i);
    float g[4];
    if (sizeof(G) == 2) {
      const uint2 raw = *reinterpret_cast<const uint2*>(grad + i);
      const bf162* gp = reinterpret_cast<const bf162*>(&raw);
      float2 a = __bfloat1622float2(gp[0]), b = __bfloat1622float2(gp[1]);
      g[0] = a.x; g[1] = a.y; g[2] = b.x; g[3] = b.y;
    } else {
      const float4 raw = *reinterpret_cast<const float4*>(grad + i);
      g[0] = raw.x; g[1] = raw.y; g[2] = raw.z; g[3] = raw.w;
    }
    float* pp = &p.x; float* pm = &mm.x; float* pv = &vv.x;
    float out[4];
#pragma unroll
    for (int k = 0; k < 4; k++) {
      const float gg = g[k] * gscale;
      float w = pp[k] * (1.f - lr * wd);
      pm[k] = b1 * pm[k] + (1.f - b1) * gg;
      pv[k] = b2 * pv[k] + (1.f - b2) * gg * gg;
      const float denom = sqrtf(pv[k]) * inv_bc2_sqrt + eps;
      w -= step * pm[k] / denom;
      pp[k] = w;
      out[k] = w;
    }
    *reinterpret_cast<float4*>(master + i) = p;
    *reinterpret_cast<float4*>(m + i) = mm;
    *reinterpret_cast<float4*>(v + i) = vv;
    uint2 packed;
    bf162* pk = reinterpret_cast<bf162*>(&packed);
    pk[0] = __floats2bfloat162_rn(out[0], out[1]);
    pk[1] = __floats2bfloat162_rn(out[2], out[3]);
    *reinterpret_cast<uint2*>(param + i) = packed;
  }
}

extern "C" int lb_adamw(void* master, void* m, void* v, const void* grad, void* param, long long n, float lr, float b1,
                        float b2, float eps, float wd, float bc1, float bc2, float gscale, int grad_fp32, void* stream) {
  if (n % 4 || n <= 0) return LB_ERR_SHAPE;
  int blocks = ew_blocks(n / 4);
  cudaStream_t s = (cudaStream_t)stream;
  if (grad_fp32)
    adamw_kernel<float><<<blocks, 256, 0, s>>>((float*)master, (float*)m, (float*)v, (const float*)grad, (bf16*)param, n,
                                               lr, b1, b2, eps, wd, bc1, bc2, gscale);
  else
    adamw_kernel<bf16><<<blocks, 256, 0, s>>>((float*)master, (float*)m, (float*)v, (const bf16*)grad, (bf16*)param, n,
                                              lr, b1, b2, eps, wd, bc1, bc2, gscale);
  LB_CHECK_LAUNCH();
  return LB_OK;
}

// out[0] += sum(x^2) (fp32).  `zero_first` clears out[0] on the stream before accumulating.
template <typename G>
__global__ void sumsq_kernel(const G* __restrict__ x, long long n, float* __restrict__ out) {
  float s = 0.f;
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (long long)gridDim.x * blockDim.x) {
    const float f = (float)x[i];
    s += f * f;
  }
  s = warp_sum(s);
  __shared__ float sh[8];
  if ((threadIdx.x & 31) == 0) sh[threadIdx.x >> 5] = s;
  __syncthreads();
  if (threadIdx.x == 0) {
    float t = 0.f;
    for (int i = 0; i < (blockDim.x >> 5); i++) t += sh[i];
    atomicAdd(out, t);
  }
}

extern "C" int lb_sumsq(const void* x, long long n, void* out, int zero_first, void* stream) {
  cudaStream_t s = (cudaStream_t)stream;
  if (zero_first) cudaMemsetAsync(out, 0, sizeof(float), s);
  sumsq_kernel<bf16><<<ew_blocks(n), 256, 0, s>>>((const bf16*)x, n, (float*)out);
  LB_CHECK_LAUNCH();
  return LB_OK;
}

__global__ void add_inplace_kernel(bf16* __restrict__ a, const bf16* __restrict__ b, long long nvec) {
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < nvec; i += (long long)gridDim.x * blockDim.x) {
    float f[8], g[8];
    unpack8(reinterpret_cast<const uint4*>(a)[i], f);
    unpack8(reinterpret_cast<const uint4*>(b)[i], g);
#pragma unroll
    for (int k = 0; k < 8; k++) f[k] += g[k];
    reinterpret_cast<uint4*>(a)[i] = pack8(f);
  }
}

extern "C" int lb_add_inplace(void* a, const void* b, long long n, void* stream) {
  if (n % 8) return LB_ERR_SHAPE;
  add_inplace_kernel<<<ew_blocks(n / 8), 256, 0, (cudaStream_t)stream>>>((bf16*)a, (const bf16*)b, n / 8);
  LB_CHECK_LAUNCH();
  return LB_OK;
}

// ---------------------------------------------------------------------------------------
// RMSNorm backward for callers that must not allocate.
//
// lb_rmsnorm_bwd() above needs a caller-provided `partial` scratch of [blocks, cols] floats.
// A caller that lives inside an allocator hook, a signal-safe teardown path, a process whose
// memory pool is frozen after start-up, or a plain C host that links this library without
// PyTorch's caching allocator has nowhere to get that buffer from, so this variant keeps the
// scratch in a fixed array in device memory that is part of the library image itself.
//
//  * Capacity: cols <= 8192 and at most 128 blocks, i.e. 4 MiB of fp32.  Every GPU on which
//    the library is loaded holds these 4 MiB until the process exits.  A larger `cols` is
//    rejected with LB_ERR_CAPACITY (-6); nothing is launched in that case.
//  * The first call on a device looks up the array's device address (cudaGetSymbolAddress,
//    with that device current) and remembers it per device.  Make that first call before
//    starting any stream capture.
//  * Nothing is allocated or freed here, by CUDA or by any library.
//  * The array is shared by every call and keeps the previous call's contents.  Each call
//    overwrites all rows that it later reads (one row per launched block), so nothing has to be
//    cleared first.  Two calls that can run at the same time on one GPU (different streams,
//    different threads) write the same rows and race: serialise them.
//  * Inputs, outputs and results are those of lb_rmsnorm_bwd; only the summation order over
//    blocks may differ (fewer, larger blocks), which changes dw by fp32 rounding only.
//  * It always runs the general kernel (row per warp, dw partial sums through shared-memory
//    atomics), not the faster block-per-row kernel that lb_rmsnorm_bwd picks for common widths:
//    that one needs one scratch row per resident block, up to 444 rows, which would not fit the
//    128 rows of the fixed array.  Expect roughly 1.5x the run time of lb_rmsnorm_bwd.
// ---------------------------------------------------------------------------------------
#define LB_STATIC_SCRATCH_MAX_COLS 8192
#define LB_STATIC_SCRATCH_MAX_BLOCKS 128
static __device__ __align__(256) float g_rmsnorm_static_scratch[LB_STATIC_SCRATCH_MAX_BLOCKS * LB_STATIC_SCRATCH_MAX_COLS];

#define LB_MAX_DEVICES 64
static float* g_static_scratch_addr[LB_MAX_DEVICES] = {nullptr};
static std::mutex g_static_scratch_mutex;     // the per-device address table is filled under this lock

extern "C" int lb_rmsnorm_bwd_static(const void* dy, const void* x, const void* w, const void* rstd, const void* dres,
                                     void* dx, void* dw, int rows, int cols, void* stream) {
  if (cols % 8 || rows <= 0) return LB_ERR_SHAPE;
  if (cols > LB_STATIC_SCRATCH_MAX_COLS) return LB_ERR_CAPACITY;
  int dev = -1;
  cudaError_t e = cudaGetDevice(&dev);
  if (e != cudaSuccess || dev < 0 || dev >= LB_MAX_DEVICES) { g_lb_last_cuda_error = (int)e; return LB_ERR_ARG; }
  float* partial = nullptr;
  {
    std::lock_guard<std::mutex> lock(g_static_scratch_mutex);
    if (g_static_scratch_addr[dev] == nullptr) {
      // In host code the array's name is only a handle; the kernel needs its device address.
      float* p = nullptr;
      e = cudaGetSymbolAddress((void**)&p, g_rmsnorm_static_scratch);
      if (e != cudaSuccess || p == nullptr) { g_lb_last_cuda_error = (int)e; return LB_ERR_LAUNCH; }
      g_static_scratch_addr[dev] = p;
    }
    partial = g_static_scratch_addr[dev];
  }
  int nblk = lb_rmsnorm_bwd_blocks(rows, cols);
  if (nblk > LB_STATIC_SCRATCH_MAX_BLOCKS) nblk = LB_STATIC_SCRATCH_MAX_BLOCKS;
  cudaStream_t s = (cudaStream_t)stream;
  size_t smem = (size_t)cols * sizeof(float);
  if (smem > 48 * 1024) cudaFuncSetAttribute(rmsnorm_bwd_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
  rmsnorm_bwd_kernel<<<nblk, 256, smem, s>>>((const bf16*)dy, (const bf16*)x, (const bf16*)w, (const float*)rstd,
                                             (const bf16*)dres, (bf16*)dx, partial, rows, cols);
  LB_CHECK_LAUNCH();
  rmsnorm_dw_reduce_kernel<<<(cols + 31) / 32, dim3(32, 32), 0, s>>>(partial, (bf16*)dw, nblk, cols);
  LB_CHECK_LAUNCH();
  return LB_OK;
}
