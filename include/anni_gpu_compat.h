/*
** The reference trainer's device API, as defined by libanni_b200.so.
**
** The reference picks its GPU backend at link time: every translation unit
** includes num/gpu.h and the linker binds the symbols either to num/gpu_stub.c
** or to num/gpu_cuda.cu.  libanni_b200.so defines the same symbol set, so it
** can take that place.  The symbols the optimizer path needs have real bodies
** on top of this library's kernels; they are declared below, each with the
** line of num/gpu.h it replaces.  Every other gpu_* symbol of that header
** (GEMM, attention, LayerNorm, cross-entropy, embedding, CUDA-graph and decode
** entry points: forward/backward, not the optimizer) is defined too and answers
** exactly like the reference's stub backend (-1, 0, NULL or nothing), which
** the reference treats as "use the CPU path".
**
** A trainer built against the reference's own num/gpu.h needs no header from
** here; this file exists for callers that do not have it (tests, bindings).
*/
#ifndef ANNI_GPU_COMPAT_H__
#define ANNI_GPU_COMPAT_H__

#include <stddef.h>

#ifdef __cplusplus
extern "C" {
#endif

/* num/real.h:3, num/vec.h:9-12, num/mat.h:12-18: layout is ABI */
typedef float ann_real_t;
typedef struct anni_vec {
	ann_real_t	*data;
	int		n;
} anni_vec;
typedef struct anni_mat {
	ann_real_t	*data;		/* host */
	ann_real_t	*d_data;	/* device twin (NULL if none) */
	int		rows;
	int		cols;
	int		on_device;	/* 0 host, 1 device, 2 synced, 3 aliased (num/mat.h:22-34) */
} anni_mat;

#define ANNI_GPU_SYNC_EAGER	0	/* num/gpu.h:17-18 */
#define ANNI_GPU_SYNC_BATCH	1
#define ANNI_GPU_PREC_FP32	0	/* num/gpu.h:23-24 */
#define ANNI_GPU_PREC_BF16	1

int	gpu_available(void);					/* gpu.h:11 */
const char	*gpu_backend_name(void);			/* gpu.h:12 */
int	gpu_mem_info(size_t *free_bytes, size_t *total_bytes);	/* gpu.h:14 */
void	gpu_set_sync_mode(int mode);				/* gpu.h:19 */
int	gpu_sync_mode(void);					/* gpu.h:20 */
void	gpu_set_compute_prec(int prec);				/* gpu.h:25 */
void	gpu_set_fp8(int on);					/* gpu.h:30 */
void	gpu_set_fp8_dgrad(int on);				/* gpu.h:31 */
int	gpu_fp8(void);						/* gpu.h:32 */
void	gpu_device_sync(void);					/* gpu.h:38 */
/* Plain cudaMalloc memory.  With ANNI_B200_COMPRESSIBLE_MALLOC=1 blocks of 8 MB and more are compressible
** device memory where the GPU offers it (anni_arena_alloc in anni_b200.h; zeroed, this device only):
** release every block with gpu_free, never cudaFree. */
void	*gpu_malloc(size_t nbytes);				/* gpu.h:40 */
void	gpu_free(void *p);					/* gpu.h:41 */
int	gpu_memcpy_h2d(void *dst, const void *src, size_t nbytes);	/* gpu.h:42 */
int	gpu_memcpy_d2h(void *dst, const void *src, size_t nbytes);	/* gpu.h:43 */
int	gpu_host_pin(void *p, size_t nbytes);			/* gpu.h:45 */
int	gpu_memcpy_d2h_async(void *dst, const void *src, size_t nbytes);	/* gpu.h:46 */
int	gpu_stream_sync(void);					/* gpu.h:47 */
int	gpu_memcpy_d2d(void *dst, const void *src, size_t nbytes);	/* gpu.h:48 */
int	gpu_memset(void *dst, int value, size_t nbytes);	/* gpu.h:49 */
void	gpu_half_wt_invalidate(const ann_real_t *fp32_dev);	/* gpu.h:56 */
void	gpu_host_forget(const void *host);			/* gpu.h:62 */
const char	*gpu_debug_last_error(void);			/* gpu.h:64 */
void	gpu_op_prof_dump(void);					/* gpu.h:66 */
void	gpu_adam_set_bf16_flat(void *bf16, const ann_real_t *fp32, int n);	/* gpu.h:71 */
int	gpu_adam_seed_bf16_flat(void *bf16, const ann_real_t *fp32, int n);	/* gpu.h:73 */
void	gpu_adam_set_weight_decay(double wd);			/* gpu.h:121 */
int	gpu_grad_sumsq(const ann_real_t *d_x, int n, double *out);	/* gpu.h:123 */
int	gpu_adam_step_dev_bf16(ann_real_t *d_param, void *d_param_bf16, ann_real_t *d_grad,
		ann_real_t *d_m, ann_real_t *d_v, int n, double lr, double beta1, double beta2,
		double eps, int t, double grad_scale);		/* gpu.h:129-132 */
/* db_host[cols] += column sums of the rows x cols device matrix x.  Done on the device, straight into the
** optimizer's gradient flat, when db_host is the host vector of a tensor attached with
** anni_lm_adam_alias_vec (anni_lm_adam.h); -1 otherwise (the caller's CPU path). */
int	gpu_mat_col_sum_add(ann_real_t *db_host, const ann_real_t *x, int rows, int cols);	/* gpu.h:198 */
int	gpu_mat_axpy(anni_mat *y, double a, const anni_mat *x);	/* gpu.h:299 */
unsigned	gpu_param_epoch(void);				/* gpu.h:346 */

/*
** Where a slice of the registered fp32 flat has its bf16 twin: the lookup the
** reference keeps private (half_wt_get, num/gpu_cuda.cu:2018-2041).  NULL when
** the pointer is outside the registered flat or no flat is registered.
*/
void	*anni_half_wt_lookup(const ann_real_t *fp32_dev, size_t n);
/*
** ANN_OP_PROF (gpu.h:66, num/gpu_cuda.cu:3205-3409): anni_op_prof_enable overrides the environment
** variable; anni_op_prof_totals waits for the device and returns the accumulated milliseconds and
** calls of one row of the table ("adam", "sumsq", "colsum", "axpy", "convert") without resetting it.
*/
void	anni_op_prof_enable(int on);
int	anni_op_prof_totals(const char *name, double *ms, long *calls);
/* 64-bit forms of the two legacy calls (the reference's `int n` stops at 2^31-1). */
int	anni_grad_sumsq64(const void *d_x, int dtype, unsigned long long n, double *out);
int	anni_adam_step_dev64(ann_real_t *d_param, void *d_param_bf16, ann_real_t *d_grad,
		ann_real_t *d_m, ann_real_t *d_v, unsigned long long n, double lr, double beta1,
		double beta2, double eps, int t, double grad_scale);

#ifdef __cplusplus
}
#endif

#endif
