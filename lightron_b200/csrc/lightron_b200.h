/* C interface of liblightron_b200.so (sm_100a).  Every function returns 0 on success or a
 * negative code: -1 bad argument, -2 CUDA launch error (see lb_last_error()), -3 unsupported
 * shape, -4 driver entry point missing, -5 tensor-map encode failed, -6 size exceeds the
 * capacity of a fixed scratch area.  Pointers are device pointers unless said otherwise;
 * `stream` is a cudaStream_t. */
#pragma once
#ifdef __cplusplus
extern "C" {
#endif

int lb_last_error(void);

/* Number of SMs of the current device. */
int lb_sm_count(void);

/* Wall-time limit (ns, default 20 s) after which a kernel that waits for a flag written by another
 * GPU gives up, sets its status word (read with the lb_*_status functions) and returns without
 * consuming the data it waited for.  Applies to later launches. */
int lb_set_flag_wait_ns(unsigned long long ns);

/* RMSNorm backward.  dy, x [rows, cols] bf16; w [cols] bf16; rstd [rows] fp32 (from the forward);
 * dres optional [rows, cols] bf16 added to dx; dx [rows, cols] bf16; dw [cols] bf16.
 * `partial` is caller-provided scratch of lb_rmsnorm_bwd_blocks(rows, cols) * cols floats. */
int lb_rmsnorm_bwd_blocks(int rows, int cols);
int lb_rmsnorm_bwd(const void* dy, const void* x, const void* w, const void* rstd, const void* dres, void* dx,
                   void* partial, void* dw, int rows, int cols, int nblk, void* stream);

/* The same operation for callers that cannot allocate device memory at call time (allocator
 * hooks, teardown paths, processes with a frozen memory pool, C hosts without a tensor
 * library).  This entry point has no counterpart in the reference project.
 * Its scratch is a fixed 4 MiB array inside the library's device image: cols must be <= 8192,
 * otherwise -6 is returned and nothing runs.  It allocates and frees nothing.  The first call on
 * each device resolves the array's device address; make it before any stream capture begins.
 * All calls share the array, so calls that may overlap on one GPU must be serialised by the
 * caller.  Same inputs and outputs as lb_rmsnorm_bwd, minus `partial` and `nblk`.  It always runs
 * the general row-per-warp kernel (the block-per-row kernel that lb_rmsnorm_bwd prefers needs more
 * scratch rows than the fixed array has), so it is slower than lb_rmsnorm_bwd, not a replacement. */
int lb_rmsnorm_bwd_static(const void* dy, const void* x, const void* w, const void* rstd, const void* dres, void* dx,
                          void* dw, int rows, int cols, void* stream);

#ifdef __cplusplus
}
#endif
