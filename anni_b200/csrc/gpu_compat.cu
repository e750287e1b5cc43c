/*
** The reference trainer's device API (num/gpu.h of the reference project) on
** top of this library's kernels, so that the trainer links libanni_b200.so in
** place of its own CUDA object.  Two parts:
**
**  - real bodies for what the optimizer path calls (memory, stream, the flat
**    bf16 twin registry, gpu_grad_sumsq, gpu_adam_step_dev_bf16, gpu_mat_axpy);
**  - "not on the device" answers for everything else, with the return values the
**    reference's stub backend gives (num/gpu_stub.c), which its callers treat
**    as "use the CPU path".
**
** All work is queued on one process-wide blocking stream, as the reference
** does (num/gpu_cuda.cu:37-44): the optimizer is called from the single
** training thread.  Errors are never fatal: -1 / NULL, and the pending CUDA
** error can be polled with gpu_debug_last_error().
*/
#include <cuda_runtime.h>
#include <math.h>
#include <stdint.h>
#include <stdio.h>
#include <stdlib.h>
#include <string.h>
#include <mutex>
#include <unordered_map>
#include "anni_gpu_compat.h"
#include "optstep_internal.h"

namespace {

std::once_flag g_once;
int g_have_gpu;
cudaStream_t g_st;
int g_sync_mode_v;
int g_prec = ANNI_GPU_PREC_FP32;
int g_fp8_on;
int g_fp8_dgrad_on;
double g_adam_wd;
unsigned g_wt_epoch;
void *g_flat_bf16;
const float *g_flat_fp32;
size_t g_flat_n;
std::mutex g_malloc_lock;	/* gpu_malloc may be entered from worker threads (gpu_cuda.cu:2644) */
std::unordered_map<void *, size_t> g_arena_blocks;	/* blocks handed out by anni_arena_alloc -> mapped size */

/* device state of the two legacy optimizer calls, created on first use */
struct legacy_state {
	anni_control	*ctl;
	int64_t		*seg_off;	/* {0, 2^62}: one tensor covering any n */
	uint32_t	*flags_twin;	/* decay + bf16 twin */
	uint32_t	*flags_plain;	/* decay only */
	float		*amax;
	int		blocks;
} g_legacy;

void init_once(void)
{
	int n = 0;

	if (cudaGetDeviceCount(&n) != cudaSuccess || n <= 0) {
		(void)cudaGetLastError();
		g_have_gpu = 0;
		return;
	}
	if (cudaStreamCreate(&g_st) != cudaSuccess) {
		g_have_gpu = 0;
		return;
	}
	g_have_gpu = 1;
}

int legacy_ready(void)
{
	static const int64_t off[2] = { 0, (int64_t)1 << 62 };
	static const uint32_t f_twin = ANNI_SEG_WD | ANNI_SEG_TWIN_BF16;
	static const uint32_t f_plain = ANNI_SEG_WD;

	if (g_legacy.ctl)
		return 0;
	if (cudaMalloc((void **)&g_legacy.ctl, sizeof(anni_control)) != cudaSuccess
	    || cudaMalloc((void **)&g_legacy.seg_off, sizeof(off)) != cudaSuccess
	    || cudaMalloc((void **)&g_legacy.flags_twin, 4) != cudaSuccess
	    || cudaMalloc((void **)&g_legacy.flags_plain, 4) != cudaSuccess
	    || cudaMalloc((void **)&g_legacy.amax, 4) != cudaSuccess
	    || cudaMemset(g_legacy.ctl, 0, sizeof(anni_control)) != cudaSuccess
	    || cudaMemcpy(g_legacy.seg_off, off, sizeof(off), cudaMemcpyHostToDevice) != cudaSuccess
	    || cudaMemcpy(g_legacy.flags_twin, &f_twin, 4, cudaMemcpyHostToDevice) != cudaSuccess
	    || cudaMemcpy(g_legacy.flags_plain, &f_plain, 4, cudaMemcpyHostToDevice) != cudaSuccess
	    || (g_legacy.blocks = anni_grid_blocks(ANNI_DT_F32, ANNI_DT_F32, 0)) < 1) {
		/* all or nothing: a half-built state must not pass for a ready one at the next call */
		(void)cudaGetLastError();
		cudaFree(g_legacy.ctl);
		cudaFree(g_legacy.seg_off);
		cudaFree(g_legacy.flags_twin);
		cudaFree(g_legacy.flags_plain);
		cudaFree(g_legacy.amax);
		memset(&g_legacy, 0, sizeof(g_legacy));
		return -1;
	}
	return 0;
}

void legacy_launch_base(anni_launch *la, uint64_t n)
{
	memset(la, 0, sizeof(*la));
	la->n = n;
	la->seg_off = g_legacy.seg_off;
	la->seg_flags = g_legacy.flags_plain;
	la->seg_amax = g_legacy.amax;
	la->seg_scale = g_legacy.amax;
	la->n_seg = 1;
	la->sc_log2 = 2;
	la->ctl = g_legacy.ctl;
}

}	/* namespace */

/* ---- device, memory, stream ------------------------------------------------ */

extern "C" int gpu_available(void)
{
	std::call_once(g_once, init_once);
	return g_have_gpu;
}

extern "C" const char *gpu_backend_name(void)
{
	return gpu_available() ? "anni_b200 (sm_100a)" : "cpu";
}

extern "C" int gpu_mem_info(size_t *free_bytes, size_t *total_bytes)
{
	size_t f = 0;
	size_t t = 0;
	int ok = gpu_available() && cudaMemGetInfo(&f, &t) == cudaSuccess;

	if (free_bytes)
		*free_bytes = ok ? f : 0;
	if (total_bytes)
		*total_bytes = ok ? t : 0;
	return ok ? 0 : -1;
}

extern "C" void gpu_set_sync_mode(int mode)
{
	g_sync_mode_v = mode;
}

extern "C" int gpu_sync_mode(void)
{
	return g_sync_mode_v;
}

extern "C" void gpu_set_compute_prec(int prec)
{
	g_prec = prec;
}

extern "C" void gpu_set_fp8(int on)
{
	g_fp8_on = on ? 1 : 0;
	g_fp8_dgrad_on = g_fp8_on;
}

extern "C" void gpu_set_fp8_dgrad(int on)
{
	g_fp8_dgrad_on = on ? 1 : 0;
}

extern "C" int gpu_fp8(void)
{
	return g_fp8_on;
}

extern "C" void gpu_device_sync(void)
{
	if (gpu_available())
		(void)cudaDeviceSynchronize();
}

/*
** Plain cudaMalloc memory, as in the reference (neither zeroed nor synchronised).  The one
** buffer that gains from compressible memory is the optimizer's gradient flat (every step
** leaves it zeroed, and zeroed lines then cost a fraction of their size on the way to HBM);
** the optimizer object of this library allocates that flat with anni_arena_alloc itself.  A
** trainer that keeps the reference's own lm_adam.c, whose flats all come from here, can opt
** in with ANNI_B200_COMPRESSIBLE_MALLOC=1: blocks of 8 MB and more then come from compressible
** memory where the device has it (zeroed, mapped for this device only: not for IPC or peer
** access).  g_arena_blocks remembers which blocks those are for gpu_free.
*/
#define ANNI_COMPRESSIBLE_FROM	((size_t)8 << 20)

static int compressible_malloc_on(void)
{
	static int on = -1;

	if (on < 0) {
		const char *e = getenv("ANNI_B200_COMPRESSIBLE_MALLOC");

		on = (e && e[0] == '1') ? 1 : 0;
	}
	return on;
}

extern "C" void *gpu_malloc(size_t nbytes)
{
	void *p = NULL;
	size_t mapped = 0;
	std::lock_guard<std::mutex> hold(g_malloc_lock);

	if (!gpu_available() || nbytes == 0)
		return NULL;
	if (compressible_malloc_on() && nbytes >= ANNI_COMPRESSIBLE_FROM
	    && anni_arena_alloc(nbytes, &p, &mapped, NULL) == ANNI_OK) {
		g_arena_blocks[p] = mapped;
		return p;
	}
	(void)cudaGetLastError();
	p = NULL;
	if (cudaMalloc(&p, nbytes) != cudaSuccess) {
		(void)cudaGetLastError();
		return NULL;
	}
	return p;
}

extern "C" void gpu_free(void *p)
{
	size_t mapped = 0;

	if (!p || !gpu_available())
		return;
	{
		std::lock_guard<std::mutex> hold(g_malloc_lock);
		auto it = g_arena_blocks.find(p);

		if (it != g_arena_blocks.end()) {
			mapped = it->second;
			g_arena_blocks.erase(it);
		}
	}
	/* the release may wait for the device: not while other threads queue for the lock */
	if (mapped)
		(void)anni_arena_free(p, mapped);
	else
		(void)cudaFree(p);
}

extern "C" int gpu_memcpy_h2d(void *dst, const void *src, size_t nbytes)
{
	if (!dst || !src || !gpu_available())
		return -1;
	return cudaMemcpyAsync(dst, src, nbytes, cudaMemcpyHostToDevice, g_st) == cudaSuccess ? 0 : -1;
}

extern "C" int gpu_memcpy_d2h(void *dst, const void *src, size_t nbytes)
{
	if (!dst || !src || !gpu_available())
		return -1;
	if (cudaMemcpyAsync(dst, src, nbytes, cudaMemcpyDeviceToHost, g_st) != cudaSuccess)
		return -1;
	return cudaStreamSynchronize(g_st) == cudaSuccess ? 0 : -1;
}

extern "C" int gpu_host_pin(void *p, size_t nbytes)
{
	cudaError_t e;

	if (!p || !gpu_available())
		return -1;
	e = cudaHostRegister(p, nbytes, cudaHostRegisterDefault);
	if (e == cudaErrorHostMemoryAlreadyRegistered) {
		(void)cudaGetLastError();
		return 0;
	}
	if (e != cudaSuccess) {
		(void)cudaGetLastError();
		return 0;	/* pageable memory still copies correctly, only slower */
	}
	return 0;
}

extern "C" int gpu_memcpy_d2h_async(void *dst, const void *src, size_t nbytes)
{
	if (!dst || !src || !gpu_available())
		return -1;
	return cudaMemcpyAsync(dst, src, nbytes, cudaMemcpyDeviceToHost, g_st) == cudaSuccess ? 0 : -1;
}

extern "C" int gpu_stream_sync(void)
{
	if (!gpu_available())
		return -1;
	return cudaStreamSynchronize(g_st) == cudaSuccess ? 0 : -1;
}

extern "C" int gpu_memcpy_d2d(void *dst, const void *src, size_t nbytes)
{
	if (!dst || !src || !gpu_available())
		return -1;
	return cudaMemcpyAsync(dst, src, nbytes, cudaMemcpyDeviceToDevice, g_st) == cudaSuccess ? 0 : -1;
}

extern "C" int gpu_memset(void *dst, int value, size_t nbytes)
{
	if (!dst || !gpu_available())
		return -1;
	return cudaMemsetAsync(dst, value, nbytes, g_st) == cudaSuccess ? 0 : -1;
}

extern "C" void gpu_host_forget(const void *host)
{
	if (host && gpu_available()) {
		/* a pinned registration must not outlive the allocation it covered */
		if (cudaHostUnregister((void *)host) != cudaSuccess)
			(void)cudaGetLastError();
	}
}

extern "C" const char *gpu_debug_last_error(void)
{
	cudaError_t e;

	if (!gpu_available())
		return "";
	e = cudaGetLastError();
	return e == cudaSuccess ? "" : cudaGetErrorString(e);
}

/*
** ANN_OP_PROF=1 (num/gpu_cuda.cu:3205-3352, 3381-3409 of the reference): device time per kind
** of operation from pairs of events recorded around each entry point of this library that
** launches work for the optimizer; the pairs are resolved, and the table printed and reset,
** by gpu_op_prof_dump, which the trainer calls once per optimizer step.
*/
namespace {

const char *const g_op_name[ANNI_OP_N] = { "adam", "sumsq", "colsum", "axpy", "convert" };
struct op_pair {
	int		op;
	cudaEvent_t	e0;
	cudaEvent_t	e1;
};
#define OP_SLOTS	1024
op_pair g_op_ev[OP_SLOTS];
int g_op_ev_made;
int g_op_ev_n;
double g_op_ms[ANNI_OP_N];
long g_op_calls[ANNI_OP_N];
int g_op_prof = -1;
std::mutex g_op_lock;

int op_prof_on(void)
{
	if (g_op_prof < 0) {
		const char *e = getenv("ANN_OP_PROF");

		g_op_prof = (e && e[0] == '1') ? 1 : 0;
	}
	return g_op_prof;
}

void op_prof_resolve(void)
{
	for (int i = 0; i < g_op_ev_n; i++) {
		float ms = 0.0f;

		if (cudaEventElapsedTime(&ms, g_op_ev[i].e0, g_op_ev[i].e1) == cudaSuccess) {
			g_op_ms[g_op_ev[i].op] += ms;
			g_op_calls[g_op_ev[i].op]++;
		} else
			(void)cudaGetLastError();
	}
	g_op_ev_n = 0;
}

}	/* namespace */

extern "C" int anni_op_begin(int op, void *stream)
{
	std::lock_guard<std::mutex> hold(g_op_lock);
	int i;

	if (!op_prof_on() || op < 0 || op >= ANNI_OP_N)
		return -1;
	if (g_op_ev_n >= OP_SLOTS) {
		/* the table is full (nobody dumped for a long while): fold what is finished */
		if (cudaDeviceSynchronize() != cudaSuccess)
			return -1;
		op_prof_resolve();
	}
	i = g_op_ev_n;
	if (i >= g_op_ev_made) {
		if (cudaEventCreate(&g_op_ev[i].e0) != cudaSuccess || cudaEventCreate(&g_op_ev[i].e1) != cudaSuccess) {
			(void)cudaGetLastError();
			return -1;
		}
		g_op_ev_made = i + 1;
	}
	g_op_ev[i].op = op;
	if (cudaEventRecord(g_op_ev[i].e0, (cudaStream_t)stream) != cudaSuccess) {
		(void)cudaGetLastError();
		return -1;
	}
	g_op_ev_n = i + 1;
	return i;
}

extern "C" void anni_op_end(int slot, void *stream)
{
	std::lock_guard<std::mutex> hold(g_op_lock);

	if (slot < 0 || slot >= g_op_ev_n)
		return;
	if (cudaEventRecord(g_op_ev[slot].e1, (cudaStream_t)stream) != cudaSuccess)
		(void)cudaGetLastError();
}

extern "C" void anni_op_prof_enable(int on)
{
	std::lock_guard<std::mutex> hold(g_op_lock);

	g_op_prof = on ? 1 : 0;
}

extern "C" int anni_op_prof_totals(const char *name, double *ms, long *calls)
{
	std::lock_guard<std::mutex> hold(g_op_lock);

	if (!name || !gpu_available())
		return -1;
	if (cudaDeviceSynchronize() != cudaSuccess)
		return -1;
	op_prof_resolve();
	for (int i = 0; i < ANNI_OP_N; i++)
		if (strcmp(name, g_op_name[i]) == 0) {
			if (ms)
				*ms = g_op_ms[i];
			if (calls)
				*calls = g_op_calls[i];
			return 0;
		}
	return -1;
}

extern "C" void gpu_op_prof_dump(void)
{
	std::lock_guard<std::mutex> hold(g_op_lock);
	double tot = 0.0;

	if (!op_prof_on() || !gpu_available())
		return;
	if (cudaDeviceSynchronize() == cudaSuccess)
		op_prof_resolve();
	for (int i = 0; i < ANNI_OP_N; i++)
		tot += g_op_ms[i];
	fprintf(stderr, "[opprof] %.3f ms of GPU op time in the optimizer's entry points, %llu kernel launches so far\n",
	    tot, (unsigned long long)anni_kernel_launches());
	for (int i = 0; i < ANNI_OP_N; i++) {
		if (g_op_calls[i] == 0)
			continue;
		fprintf(stderr, "[opprof]   %-11s %8.3f ms %5.1f%% %6ld calls %8.3f ms/call\n", g_op_name[i],
		    g_op_ms[i], tot > 0.0 ? 100.0 * g_op_ms[i] / tot : 0.0, g_op_calls[i],
		    g_op_ms[i] / (double)g_op_calls[i]);
		g_op_ms[i] = 0.0;
		g_op_calls[i] = 0;
	}
}

/* ---- the flat bf16 twin registry ---------------------------------------------- */

extern "C" void gpu_half_wt_invalidate(const ann_real_t *fp32_dev)
{
	(void)fp32_dev;
	g_wt_epoch++;	/* derived copies (packed QKV, fp8, host-vector caches) rebuild lazily */
}

extern "C" unsigned gpu_param_epoch(void)
{
	return g_wt_epoch;
}

extern "C" void gpu_adam_set_bf16_flat(void *bf16, const ann_real_t *fp32, int n)
{
	g_flat_bf16 = bf16;
	g_flat_fp32 = fp32;
	g_flat_n = bf16 && fp32 && n > 0 ? (size_t)n : 0;
}

extern "C" int gpu_adam_seed_bf16_flat(void *bf16, const ann_real_t *fp32, int n)
{
	if (!bf16 || !fp32 || n <= 0 || !gpu_available())
		return -1;
	{
		const int slot = anni_op_begin(ANNI_OP_CONVERT, g_st);
		const int rc = anni_launch_f32_to_bf16((uint16_t *)bf16, fp32, (uint64_t)n, g_st);

		anni_op_end(slot, g_st);
		return rc == ANNI_OK ? 0 : -1;
	}
}

extern "C" void *anni_half_wt_lookup(const ann_real_t *fp32_dev, size_t n)
{
	size_t off;

	if (!g_flat_n || !fp32_dev || fp32_dev < g_flat_fp32)
		return NULL;
	off = (size_t)(fp32_dev - g_flat_fp32);
	if (off >= g_flat_n || n > g_flat_n - off)
		return NULL;
	return (char *)g_flat_bf16 + off * 2;	/* same element offset, two bytes each */
}

/* ---- the optimizer's two device calls ------------------------------------------ */

extern "C" void gpu_adam_set_weight_decay(double wd)
{
	g_adam_wd = wd > 0.0 ? wd : 0.0;
}

extern "C" int anni_grad_sumsq64(const void *d_x, int dtype, unsigned long long n, double *out)
{
	anni_launch la;

	if (!d_x || n == 0 || !out || !gpu_available() || legacy_ready() != 0)
		return -1;
	if (dtype != ANNI_DT_F32 && dtype != ANNI_DT_BF16)
		return -1;
	legacy_launch_base(&la, n);
	la.grad = (void *)d_x;
	la.aligned = ((uintptr_t)d_x & 15) == 0;
	{
		const int slot = anni_op_begin(ANNI_OP_SUMSQ, g_st);
		const int rc = anni_launch_norm(&la, dtype, ANNI_DT_F32, g_legacy.blocks, g_st);

		anni_op_end(slot, g_st);
		if (rc != ANNI_OK)
			return -1;
	}
	/* the reference returns the sum to the host with a blocking copy (gpu_cuda.cu:8532) */
	if (cudaMemcpyAsync(out, (char *)g_legacy.ctl + offsetof(anni_control, reduce), sizeof(double),
	    cudaMemcpyDeviceToHost, g_st) != cudaSuccess)
		return -1;
	return cudaStreamSynchronize(g_st) == cudaSuccess ? 0 : -1;
}

extern "C" int gpu_grad_sumsq(const ann_real_t *d_x, int n, double *out)
{
	if (n <= 0)
		return -1;
	return anni_grad_sumsq64(d_x, ANNI_DT_F32, (unsigned long long)n, out);
}

extern "C" int anni_adam_step_dev64(ann_real_t *d_p, void *d_p_bf16, ann_real_t *d_g, ann_real_t *d_m,
	ann_real_t *d_v, unsigned long long n, double lr, double beta1, double beta2, double eps, int t,
	double grad_scale)
{
	anni_launch la;
	anni_optstep_hyper hp;
	const int twin = d_p_bf16 && g_prec == ANNI_GPU_PREC_BF16;

	if (!d_p || !d_g || !d_m || !d_v || n == 0 || !(lr > 0.0) || t < 1)
		return -1;
	if (!gpu_available() || legacy_ready() != 0)
		return -1;
	legacy_launch_base(&la, n);
	la.master = d_p;
	la.m = d_m;
	la.v = d_v;
	la.grad = d_g;
	la.twin16 = twin ? (uint16_t *)d_p_bf16 : NULL;
	la.seg_flags = twin ? g_legacy.flags_twin : g_legacy.flags_plain;
	la.aligned = (((uintptr_t)d_p | (uintptr_t)d_g | (uintptr_t)d_m | (uintptr_t)d_v
	    | (uintptr_t)la.twin16) & 15) == 0;
	memset(&hp, 0, sizeof(hp));
	hp.lr = lr;
	hp.beta1 = beta1;
	hp.beta2 = beta2;
	hp.eps = eps;
	hp.weight_decay = g_adam_wd;
	hp.grad_clip = 0.0;		/* the caller folded its clip factor into grad_scale */
	hp.grad_scale = grad_scale;
	hp.t = t;
	/* "d_grad is zeroed after" (gpu.h:125-127); with fp32 moments the double update term costs a few per cent */
	hp.flags = ANNI_STEP_ZERO_GRAD | ANNI_STEP_EXACT_UPDATE;
	if (anni_fill_hyper(&la, &hp) != ANNI_OK)
		return -1;		/* bias correction not positive, as gpu_cuda.cu:8681 */
	la.flags |= ANNI_LAUNCH_HOST_COEF;
	{
		const int slot = anni_op_begin(ANNI_OP_ADAM, g_st);
		const int rc = anni_launch_update(&la, ANNI_DT_F32, ANNI_DT_F32, g_legacy.blocks, g_st);

		anni_op_end(slot, g_st);
		return rc == ANNI_OK ? 0 : -1;
	}
}

extern "C" int gpu_adam_step_dev_bf16(ann_real_t *d_p, void *d_p_bf16, ann_real_t *d_g,
	ann_real_t *d_m, ann_real_t *d_v, int n, double lr, double beta1, double beta2, double eps,
	int t, double grad_scale)
{
	if (n <= 0)
		return -1;
	return anni_adam_step_dev64(d_p, d_p_bf16, d_g, d_m, d_v, (unsigned long long)n, lr, beta1,
	    beta2, eps, t, grad_scale);
}

/* y += a x on the device twins (gpu.h:299); host-authoritative operands are uploaded first. */
extern "C" int gpu_mat_axpy(anni_mat *y, double a, const anni_mat *x)
{
	size_t n;
	size_t nb;
	anni_mat *xm = (anni_mat *)x;
	anni_mat *ops[2];

	if (!y || !x || y->rows != x->rows || y->cols != x->cols || !gpu_available())
		return -1;
	n = (size_t)y->rows * (size_t)y->cols;
	nb = n * sizeof(float);
	if (n == 0)
		return -1;
	ops[0] = y;
	ops[1] = xm;
	for (int k = 0; k < 2; k++) {
		anni_mat *mt = ops[k];

		if (!mt->d_data) {
			mt->d_data = (float *)gpu_malloc(nb);
			if (!mt->d_data)
				return -1;
			mt->on_device = 0;
		}
		if (mt->on_device == 0) {	/* host is authoritative: bring it over */
			if (!mt->data || gpu_memcpy_h2d(mt->d_data, mt->data, nb) != 0)
				return -1;
			mt->on_device = 2;
		}
	}
	{
		const int slot = anni_op_begin(ANNI_OP_AXPY, g_st);
		const int rc = anni_launch_axpy(y->d_data, x->d_data, (float)a, n, g_st);

		anni_op_end(slot, g_st);
		if (rc != ANNI_OK)
			return -1;
	}
	if (y->on_device != 3)
		y->on_device = 1;	/* device-authoritative; an aliased view stays aliased */
	if (g_sync_mode_v == ANNI_GPU_SYNC_EAGER)
		(void)cudaStreamSynchronize(g_st);
	return 0;
}

/* ---- bias / LayerNorm gradients that never leave the device -------------------------- */

/*
** The reference accumulates the column sums that make a bias gradient in a device buffer keyed
** by the HOST gradient vector and adds them into that vector at the next device sync
** (colsum_acc, num/gpu_cuda.cu:3130-3195), from where the optimizer uploads them again each
** step (seg_gather, lang/lm_adam.c:361-396).  Here the optimizer object registers, per vector
** tensor, the slice of its device gradient flat that stands for the host vector
** (anni_lm_adam_alias_vec): gpu_mat_col_sum_add then adds straight into the flat and the
** gradient never travels.  Unregistered vectors answer -1, "use the CPU path", as before.
*/
namespace {

struct colsum_slot {
	const ann_real_t	*host;
	float			*dev;
	int			cols;
};
#define COLSUM_SLOTS	1024
colsum_slot g_colsum[COLSUM_SLOTS];
int g_colsum_n;
std::mutex g_colsum_lock;

/* out[c] += sum over rows of x[r][c]: one block per 32 columns, eight row lanes, fixed order */
__global__ void __launch_bounds__(256) colsum_add_kernel(float *out, const float *x, int rows, int cols)
{
	__shared__ float part[8][33];
	const int lane = threadIdx.x & 31;
	const int rg = threadIdx.x >> 5;
	const int c = blockIdx.x * 32 + lane;
	float acc = 0.0f;

	if (c < cols)
		for (int r = rg; r < rows; r += 8)
			acc += x[(size_t)r * cols + c];
	part[rg][lane] = acc;
	__syncthreads();
	if (rg == 0 && c < cols) {
		float t = part[0][lane];

		for (int k = 1; k < 8; k++)
			t += part[k][lane];
		out[c] += t;
	}
}

}	/* namespace */

extern "C" int anni_colsum_register(const ann_real_t *host, float *dev, int cols)
{
	std::lock_guard<std::mutex> hold(g_colsum_lock);

	if (!host || !dev || cols <= 0)
		return -1;
	for (int i = 0; i < g_colsum_n; i++)
		if (g_colsum[i].host == host) {
			g_colsum[i].dev = dev;
			g_colsum[i].cols = cols;
			return 0;
		}
	if (g_colsum_n >= COLSUM_SLOTS)
		return -1;
	g_colsum[g_colsum_n].host = host;
	g_colsum[g_colsum_n].dev = dev;
	g_colsum[g_colsum_n].cols = cols;
	g_colsum_n++;
	return 0;
}

extern "C" void anni_colsum_forget(const void *dev_lo, const void *dev_hi)
{
	std::lock_guard<std::mutex> hold(g_colsum_lock);
	int k = 0;

	for (int i = 0; i < g_colsum_n; i++)
		if ((const void *)g_colsum[i].dev < dev_lo || (const void *)g_colsum[i].dev >= dev_hi)
			g_colsum[k++] = g_colsum[i];
	g_colsum_n = k;
}

extern "C" int gpu_mat_col_sum_add(ann_real_t *db_host, const ann_real_t *x, int rows, int cols)	/* gpu.h:198 */
{
	cudaPointerAttributes at;
	float *dev = NULL;

	if (!db_host || !x || rows <= 0 || cols <= 0 || !gpu_available())
		return -1;
	{
		std::lock_guard<std::mutex> hold(g_colsum_lock);

		for (int i = 0; i < g_colsum_n; i++)
			if (g_colsum[i].host == db_host && g_colsum[i].cols == cols)
				dev = g_colsum[i].dev;
	}
	if (!dev)
		return -1;	/* not a registered gradient vector: the caller's CPU path */
	if (cudaPointerGetAttributes(&at, x) != cudaSuccess || at.type != cudaMemoryTypeDevice) {
		(void)cudaGetLastError();
		return -1;	/* the matrix must already be on the device */
	}
	{
		const int slot = anni_op_begin(ANNI_OP_COLSUM, g_st);

		colsum_add_kernel<<<(cols + 31) / 32, 256, 0, g_st>>>(dev, x, rows, cols);
		anni_count_launch();
		anni_op_end(slot, g_st);
	}
	if (cudaGetLastError() != cudaSuccess)
		return -1;
	if (g_sync_mode_v == ANNI_GPU_SYNC_EAGER)
		(void)cudaStreamSynchronize(g_st);
	return 0;
}

/* ---- everything else in num/gpu.h: not on the device ----------------------------- */

/*
** Forward/backward, inference and CUDA-graph entry points.  Only the symbol
** and the value it returns matter to the linker and to the callers (they fall
** back to their CPU code); argument lists are therefore left empty.  Values
** are those of the reference's stub backend.
*/
#define NOT_ON_DEVICE(name)	extern "C" int name() { return -1; }
#define ANSWERS_ZERO(name)	extern "C" int name() { return 0; }
#define NO_POINTER(name)	extern "C" void *name() { return NULL; }
#define NOTHING_TO_DO(name)	extern "C" void name() { }

NOT_ON_DEVICE(gpu_ce_fetch_mean)
NOT_ON_DEVICE(gpu_mat_mul)
NOT_ON_DEVICE(gpu_mat_mul_bias)
NOT_ON_DEVICE(gpu_mat_mul_res)
NOT_ON_DEVICE(gpu_mat_mul_bias_relu)
NOT_ON_DEVICE(gpu_mat_mul_bt)
NOT_ON_DEVICE(gpu_mat_mul_bt_acc)
NOT_ON_DEVICE(gpu_mat_mul_bt_twin)
NOT_ON_DEVICE(gpu_mat_mul_at)
NOT_ON_DEVICE(gpu_mat_outer_add)
NOT_ON_DEVICE(gpu_layernorm_backward)
NOT_ON_DEVICE(gpu_layernorm_backward_acc)
NOT_ON_DEVICE(gpu_layernorm_backward_x)
NOT_ON_DEVICE(gpu_layernorm_xhat)
NOT_ON_DEVICE(gpu_softmax_rows)
NOT_ON_DEVICE(gpu_softmax_bwd_rows)
NOT_ON_DEVICE(gpu_layernorm_forward_ex)
NOT_ON_DEVICE(gpu_bias_row_add)
NOT_ON_DEVICE(gpu_ce_delta_from_softmax)
NOT_ON_DEVICE(gpu_ce_softmax_delta_bf16)
ANSWERS_ZERO(gpu_ce_bias_fused)
NOT_ON_DEVICE(gpu_ce_bf16_delta_done)
NOT_ON_DEVICE(gpu_ce_nll_rows)
NOT_ON_DEVICE(gpu_posenc_add_packed)
NOT_ON_DEVICE(gpu_relu_backward)
NOT_ON_DEVICE(gpu_ffn_relu_bwd_fused)
ANSWERS_ZERO(gpu_act_bf16_only)
NOT_ON_DEVICE(gpu_attn_causal_fwd)
NOT_ON_DEVICE(gpu_attn_flash_fwd)
NOT_ON_DEVICE(gpu_attn_fa_fwd)
ANSWERS_ZERO(gpu_attn_fa_usable)
NOT_ON_DEVICE(gpu_attn_fa_bwd)
extern "C" int gpu_attn_qkv_bwd() { return 1; }	/* the stub's "not handled" answer for this call */
NOT_ON_DEVICE(gpu_attn_tiled_bwd)
NOT_ON_DEVICE(gpu_attn_causal_bwd)
NOT_ON_DEVICE(gpu_attn_tc_fwd)
NOT_ON_DEVICE(gpu_attn_tc_bwd)
NOT_ON_DEVICE(gpu_attn_qkv_fused)
NOT_ON_DEVICE(gpu_pack_seq_rows)
NOT_ON_DEVICE(gpu_unpack_seq_rows)
NOT_ON_DEVICE(gpu_ffn_w1_finish)
NOT_ON_DEVICE(gpu_mat_copy)
NOT_ON_DEVICE(gpu_mat_add)
NOT_ON_DEVICE(gpu_mat_add2)
NOT_ON_DEVICE(gpu_embed_lookup)
NOT_ON_DEVICE(gpu_embed_scatter)
NOT_ON_DEVICE(gpu_graph_begin)
NOT_ON_DEVICE(gpu_graph_end)
NOT_ON_DEVICE(gpu_graph_replay)
ANSWERS_ZERO(gpu_graph_replayable)
ANSWERS_ZERO(gpu_graph_supported)
NOT_ON_DEVICE(gpu_ids_stage)
NOT_ON_DEVICE(gpu_dec_set_layer)
NOT_ON_DEVICE(gpu_dec_set_io)
NOT_ON_DEVICE(gpu_dec_kv_load)
NOT_ON_DEVICE(gpu_dec_step)
NO_POINTER(gpu_host_alloc)
NO_POINTER(gpu_copy_stream)
NO_POINTER(gpu_ce_targets_staged)
NO_POINTER(gpu_dec_create)
NOTHING_TO_DO(gpu_grad_twins_clear)
NOTHING_TO_DO(gpu_attn_qkv_bf16_hint)
NOTHING_TO_DO(gpu_attn_set_seqlens)
NOTHING_TO_DO(gpu_host_free)
NOTHING_TO_DO(gpu_graph_destroy)
NOTHING_TO_DO(gpu_graph_set_mode)
NOTHING_TO_DO(gpu_ids_unstage)
NOTHING_TO_DO(gpu_dec_free)
